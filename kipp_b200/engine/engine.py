"""The engine as Python sees it: a face of the host core (csrc/host/engine.hpp).

``step`` takes a batch of (request, its next tokens), portions of prompts
beside single decoded tokens, cut anywhere; the library runs exactly those
tokens as one batch against the cache that earlier steps left and returns the
logits at the wanted places.  It generalises the reference's ``kipp_eval_batch``
(src/kipp.c:3984-4082): any mixture of items, nothing changes on error, lengths
advance on success.

What this module adds to the C interface: requests named by any hashable
object, device memory of the library wrapped as torch tensors, tensors handed
over from torch (a dict of tensors, or random weights made on the device one at
a time), and the calls back into parts that are defined in Python.
"""
from __future__ import annotations

import ctypes
import json
from typing import Iterable, Optional

import torch

from .. import native as N
from ..cache import CacheManager
from ..cache import _native as cache_native
from ..config.base import ConfigError, ModelConfig, read_config_json
from ..config.registry import get_architecture, is_registered
from ..models.spec import LayerRun, ModelSpec
from ..parts.base import PagedKVSpec
from ..weights.loader import Checkpoint, storage_dtype
from ..weights.random_init import random_tensors
from .batch import StepEntry
from .runtime import parse_dtype

_TYPESTR = {torch.float32: "<f4", torch.int32: "<i4", torch.bfloat16: "<i2", torch.float16: "<f2",
            torch.int64: "<i8", torch.uint8: "|u1", torch.float64: "<f8"}
_DTYPE_CODE = {torch.float32: N.DTYPE_F32, torch.bfloat16: N.DTYPE_BF16, torch.float16: N.DTYPE_F16,
               torch.int32: N.DTYPE_I32, torch.int64: N.DTYPE_I64, torch.int16: N.DTYPE_I16,
               torch.int8: N.DTYPE_I8, torch.uint8: N.DTYPE_U8}
_CODE_DTYPE = {N.DTYPE_F32: torch.float32, N.DTYPE_BF16: torch.bfloat16, N.DTYPE_I32: torch.int32}


class _DeviceMemory:
    """Library-owned device memory, described the way torch can adopt it."""

    def __init__(self, ptr: int, shape: tuple, typestr: str, owner):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}
        self._owner = owner


def device_tensor(ptr: int, shape: tuple, dtype: torch.dtype, device: torch.device, owner=None) -> torch.Tensor:
    """A torch tensor over device memory the library owns (no copy)."""
    n = 1
    for d in shape:
        n *= int(d)
    if n == 0 or not ptr:
        return torch.empty(shape, dtype=dtype, device=device)
    t = torch.as_tensor(_DeviceMemory(ptr, shape, _TYPESTR[dtype], owner), device=device)
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


class _Runtime:
    """What code outside the library asks of an engine's device side."""

    def __init__(self, engine: "Engine"):
        self._engine = engine
        self.device = engine.device
        self.dtype = engine.dtype

    def check_status(self) -> None:
        self._engine.synchronize()


class _ExternalMeta:
    pass


class ExternalContext:
    """What a part defined in Python sees of a step: the metadata as tensors on
    the device and as host lists, the compute dtype, and its per-request state."""

    def __init__(self, engine: "Engine", part, call: N.ExternalCall):
        dev = engine.device
        self.engine = engine
        self.device = dev
        self.dtype = engine.dtype
        self._part = part
        self._call = call
        T, n = call.tokens, call.entries
        m = _ExternalMeta()
        m.tokens, m.entries = T, n
        m.token_ids = device_tensor(call.token_ids, (T,), torch.int32, dev)
        m.positions = device_tensor(call.positions, (T,), torch.int32, dev)
        m.entry_of_token = device_tensor(call.entry_of_token, (T,), torch.int32, dev)
        m.q_start = device_tensor(call.q_start, (n + 1,), torch.int32, dev)
        m.context_len = device_tensor(call.context_len, (n,), torch.int32, dev)
        m.slots = device_tensor(call.slots, (n,), torch.int32, dev)
        m.q_lens = [call.host_q_lens[i] for i in range(n)]
        m.starts = [call.host_context_len[i] for i in range(n)]
        m.kv_lens = [s + q for s, q in zip(m.starts, m.q_lens)]
        m.host_slots = [call.host_slots[i] for i in range(n)]
        self.meta = m

    def state_view(self, run=None) -> torch.Tensor:
        """``[max_requests, *shape]`` state of the run this call is for; index it
        with ``meta.slots``."""
        spec = self._part.state_spec()
        if spec is None or not self._call.state:
            raise RuntimeError("this part declared no per-request state")
        return device_tensor(self._call.state, (self._call.max_requests,) + tuple(spec.shape), spec.dtype, self.device)


class _LazyRandom(dict):
    """Mapping name -> random tensor made on first access and not kept, so that
    a large model never exists twice."""

    def __init__(self, specs, seed, sigma, norm_jitter, dtype, device):
        super().__init__()
        self._specs = {s.name: s for s in specs}
        self._args = (seed, sigma, norm_jitter, dtype, device)

    def __contains__(self, name) -> bool:
        s = self._specs.get(name)
        return s is not None and not (s.optional and s.alias_of is not None)

    def get(self, name, default=None):
        return self[name] if name in self else default

    def __getitem__(self, name):
        seed, sigma, jitter, dtype, device = self._args
        s = self._specs[name]
        for _, t in random_tensors([s], seed, sigma=sigma, norm_jitter=jitter, dtype=dtype,
                                   device=device, skip_aliased=False):
            return t
        raise KeyError(name)


class _CheckpointTensors:
    """Mapping name -> CPU tensor (storage dtype) over a model folder, for the
    parts defined in Python (the library reads its own parts' tensors itself)."""

    def __init__(self, folder: str):
        self._ckpt = Checkpoint(folder)

    def __contains__(self, name) -> bool:
        return name in self._ckpt

    def __getitem__(self, name):
        if name not in self._ckpt:
            raise KeyError(name)
        t = self._ckpt.tensor(name)
        return t.to(storage_dtype(t.dtype))

    def get(self, name, default=None):
        return self[name] if name in self else default


class Engine:
    def __init__(self, spec: ModelSpec, tensors, *, folder: Optional[str] = None, dtype="bfloat16",
                 device: str | torch.device = "cuda:0", page_size: int = 16,
                 cache_tokens: Optional[int] = 8192, max_requests: int = 64, max_batch_tokens: int = 8192,
                 max_logit_rows: Optional[int] = None, cuda_graphs: bool = True, kv_round_bf16: bool = False,
                 own_length_splits: bool = False):
        """``tensors`` maps checkpoint names to torch tensors (CPU or CUDA); with
        ``folder`` the library reads the model folder itself.  ``cache_tokens``
        None sizes the cache from the free device memory."""
        self.spec = spec
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("kipp_b200 runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; kipp_b200 has no CPU fallback")
        self.dtype = parse_dtype(dtype)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_batch_tokens = max_batch_tokens
        self._lib = N.lib()
        self._h = None
        self._owners = cache_native.OwnerIds()
        self._callback_error: Optional[BaseException] = None
        self._keep: list = []
        opt = N.EngineOptions()
        self._lib.kipp_engine_default_options(ctypes.byref(opt))
        opt.dtype = _DTYPE_CODE[self.dtype]
        opt.device = self.device.index or 0
        opt.page_size = page_size
        opt.cache_tokens = int(cache_tokens or 0)
        opt.max_requests = max_requests
        opt.max_batch_tokens = max_batch_tokens
        opt.max_logit_rows = int(max_logit_rows or 0)
        opt.cuda_graphs = 1 if cuda_graphs else 0
        opt.kv_round_bf16 = 1 if kv_round_bf16 else 0
        opt.own_length_splits = 1 if own_length_splits else 0
        plan, external = spec.to_plan()
        self._external = external
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            ext_array, n_ext = self._external_array(external)
            if folder is not None and not external and spec.plan is not None:
                # an architecture of the library's own, from a folder: nothing of Python's in between
                rc = self._lib.kipp_engine_open(folder.encode(), ctypes.byref(opt), ctypes.byref(handle))
            elif folder is not None:
                rc = self._lib.kipp_engine_create(json.dumps(plan).encode(), folder.encode(),
                                                  ctypes.cast(None, N.TENSOR_PROVIDER), None, ext_array, n_ext,
                                                  ctypes.byref(opt), ctypes.byref(handle))
            else:
                provider = self._provider(tensors)
                rc = self._lib.kipp_engine_create(json.dumps(plan).encode(), None, provider, None, ext_array, n_ext,
                                                  ctypes.byref(opt), ctypes.byref(handle))
            self._provider_keep = None
            if self._callback_error is not None:
                err, self._callback_error = self._callback_error, None
                raise err
            N.check(rc)
            self._h = handle
            self._stream = torch.cuda.ExternalStream(self._lib.kipp_engine_stream(handle), device=self.device)
            runtime = _Runtime(self)
            source = _CheckpointTensors(folder) if folder is not None else tensors
            for part, prefix in external:
                with torch.cuda.stream(self._stream):
                    part.bind(source, prefix, runtime)
            self._stream.synchronize()
        self.runtime = _Runtime(self)
        info = self.info()
        self.vocab_size = info["vocab_size"]
        groups = [(PagedKVSpec(g["kv_heads"], g["head_dim"], g["window"]), g["caches"], g["pages"])
                  for g in info["cache_groups"]]
        self.cache = CacheManager.view_of(self._lib.kipp_engine_cache_manager(self._h), groups, page_size,
                                          max_requests, self._owners, keep=self)
        self.states = {s["cache"]: s["bytes_per_request"] for s in info["states"]}
        self.cuda_graphs = bool(info["cuda_graphs"])

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.kipp_engine_close(h)
            self._h = None

    # -- construction ------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str, **options) -> "Engine":
        """Load ``folder/config.json`` and its safetensors; the model class is
        chosen by ``architectures[0]``: an architecture registered from Python if
        there is one of that name, else the library's own registry."""
        data = read_config_json(folder)
        archs = data.get("architectures") if isinstance(data, dict) else None
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json lacks 'architectures': [name]")
        arch = get_architecture(archs[0])         # raises ConfigError for a name nobody knows
        config = arch.config_class.from_dict(data)
        spec = arch.build(config)
        return cls(spec, None, folder=folder, **options)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int, *, sigma: Optional[float] = None,
                    norm_jitter: float = 0.1, weight_dtype: torch.dtype = torch.bfloat16,
                    **options) -> "Engine":
        """Random weights made on the device (no files): for benchmarks of
        sizes too large to write out."""
        spec = get_architecture(config.architecture).build(config)
        device = options.get("device", "cuda:0")
        if sigma is None:
            sigma = float(getattr(config, "initializer_range", 0.02))
        tensors = _LazyRandom(spec.tensor_specs(), seed, sigma, norm_jitter, weight_dtype, device)
        return cls(spec, tensors, **options)

    def _provider(self, tensors):
        def provide(_user, name, view):
            try:
                t = tensors.get(name.decode()) if hasattr(tensors, "get") else None
                if t is None:
                    return 1
                if t.dtype not in _DTYPE_CODE:
                    t = t.float()
                t = t.contiguous()
                if t.is_cuda:
                    torch.cuda.current_stream(t.device).synchronize()
                self._provider_keep = t                    # alive until the next call
                v = view.contents
                v.data = t.data_ptr()
                v.on_device = 1 if t.is_cuda else 0
                v.dtype = _DTYPE_CODE[t.dtype]
                v.ndim = t.dim()
                for i, d in enumerate(t.shape):
                    v.shape[i] = d
                return 0
            except BaseException as e:                     # noqa: BLE001 - crosses a C frame
                self._callback_error = e
                return 1
        cb = N.TENSOR_PROVIDER(provide)
        self._keep.append(cb)
        return cb

    def _external_array(self, external):
        if not external:
            return None, 0
        arr = (N.ExternalPart * len(external))()
        for i, (part, _prefix) in enumerate(external):
            cb = N.EXTERNAL_FORWARD(self._make_forward(part))
            self._keep.append(cb)
            arr[i].user = None
            arr[i].forward = cb
        self._keep.append(arr)
        return arr, len(external)

    def _make_forward(self, part):
        def forward(_user, call_ptr):
            try:
                c = call_ptr.contents
                ctx = ExternalContext(self, part, c)
                dev, T = self.device, c.tokens
                with torch.cuda.stream(self._stream):
                    residual = device_tensor(c.residual, (T, c.hidden), torch.float32, dev)
                    h = None
                    if c.input:
                        h = device_tensor(c.input, (T, c.input_cols), _CODE_DTYPE[c.input_dtype], dev)
                    if c.role == 2:
                        part.forward(ctx, LayerRun(c.layer, c.cache, bool(c.writes_cache)), h, residual)
                    elif c.role == 3:
                        part.forward(ctx, h, residual)
                    elif c.role == 0:
                        part.forward(ctx, residual)
                    elif c.role == 1:
                        n_rows = c.n_rows
                        rows = device_tensor(c.rows, (n_rows,), torch.int32, dev) if c.rows else None
                        out = device_tensor(c.output, (n_rows, c.hidden), self.dtype, dev)
                        part.forward(ctx, residual, out, rows, n_rows)
                    else:
                        raise RuntimeError(f"unknown role {c.role}")
                return 0
            except BaseException as e:                     # noqa: BLE001 - crosses a C frame
                self._callback_error = e
                return 1
        return forward

    @property
    def stream(self) -> torch.cuda.Stream:
        """The CUDA stream the engine's kernels run on (events that time its work are
        recorded there)."""
        return self._stream

    # -- requests ------------------------------------------------------------------
    def _id(self, rid, create: bool = False) -> int:
        i = self._owners.id_of(rid, create=create)
        if not i:
            raise KeyError(rid)
        return i

    def _check(self, rc: int) -> None:
        if self._callback_error is not None:
            err, self._callback_error = self._callback_error, None
            raise err
        N.check(rc, engine=self._h)

    def _forget_dead(self, rids) -> None:
        for r in rids:
            i = self._owners.id_of(r)
            if i and not self._lib.kipp_engine_is_live(self._h, i):
                self._owners.forget(r)

    def add_request(self, rid) -> int:
        if rid in self._owners:
            raise ValueError(f"request {rid!r} is already live")
        try:
            self._check(self._lib.kipp_engine_add_request(self._h, self._id(rid, create=True)))
        except Exception:
            self._forget_dead([rid])
            raise
        return self.cache.slot(rid)

    def finish(self, rid) -> None:
        """The request is over: its pages and its slot are given back."""
        self._check(self._lib.kipp_engine_finish(self._h, self._id(rid)))
        self._owners.forget(rid)

    def truncate(self, rid, new_length: int) -> None:
        """Cut a live request back to its first ``new_length`` tokens; the pages
        beyond go back.  A model whose mixers keep state per request can only be
        cut back to nothing (the state is then cleared): a state cannot be unwound."""
        self._check(self._lib.kipp_engine_truncate(self._h, self._id(rid), int(new_length)))

    def reset(self, rid) -> None:
        """The request keeps its slot and starts again from an empty context."""
        self.truncate(rid, 0)

    def length(self, rid) -> int:
        return self._lib.kipp_engine_length(self._h, self._id(rid))

    def is_live(self, rid) -> bool:
        i = self._owners.id_of(rid)
        return bool(i) and bool(self._lib.kipp_engine_is_live(self._h, i))

    # -- the step ----------------------------------------------------------------------
    def _entries(self, entries):
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        n = len(entries)
        arr = (N.StepEntryC * max(n, 1))()
        keep = []
        for i, e in enumerate(entries):
            toks = (ctypes.c_int32 * max(len(e.tokens), 1))(*[int(t) for t in e.tokens])
            want = (ctypes.c_int32 * max(len(e.want), 1))(*[int(w) for w in e.want])
            keep += [toks, want]
            arr[i].request = self._id(e.request, create=True)
            arr[i].tokens, arr[i].n_tokens = toks, len(e.tokens)
            arr[i].want, arr[i].n_want = want, len(e.want)
        return entries, arr, keep

    def step(self, entries: Iterable[StepEntry], *, check: bool = False) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits ``[wanted, vocab]`` on the
        device in the order of the entries and of their ``want`` lists (None if
        nothing is wanted).  The tensor is the engine's memory: read or copy it
        before the next step.  Raises ``OutOfPages`` with no request changed
        when the cache cannot hold the step."""
        entries, arr, keep = self._entries(entries)
        if not entries:
            return None
        logits, rows = ctypes.c_void_p(), ctypes.c_int()
        with torch.cuda.device(self.device):
            self._stream.wait_stream(torch.cuda.current_stream())
            rc = self._lib.kipp_engine_step(self._h, arr, len(entries), ctypes.byref(logits), ctypes.byref(rows))
            try:
                self._check(rc)
            except Exception:
                self._forget_dead([e.request for e in entries])
                raise
            torch.cuda.current_stream().wait_stream(self._stream)
            if check:
                self.synchronize()
        del keep
        if not logits.value or rows.value == 0:
            return None
        return device_tensor(logits.value, (rows.value, self.vocab_size), torch.float32, self.device, owner=self)

    def last_logits(self):
        """The logits of the last step as a float32 array ``[rows, vocab]`` on the host
        (None when it wanted none)."""
        import numpy as np
        rows = self._lib.kipp_engine_last_rows(self._h)
        if rows <= 0:
            return None
        out = np.empty((rows, self.vocab_size), dtype=np.float32)
        self._check(self._lib.kipp_engine_read_logits(self._h, out.ctypes.data, out.size))
        return out

    def _debug_set_status(self, word: int, value: int) -> None:
        self._check(self._lib.kipp_engine_debug_set_status(self._h, word, value))

    def synchronize(self) -> None:
        """Wait for the engine's stream and raise if a kernel refused an access or
        gave up a wait."""
        self._check(self._lib.kipp_engine_synchronize(self._h))

    def profile_start(self) -> None:
        """From here on steps run without CUDA graphs and every kernel launch is followed
        by an event on the engine's stream (see :meth:`profile_stop`)."""
        self._check(self._lib.kipp_engine_profile(self._h, 1))

    def profile_stop(self) -> dict:
        """{kernel name: milliseconds} since :meth:`profile_start`: the time between
        consecutive events, so the gaps between launches are inside; read as shares."""
        self._check(self._lib.kipp_engine_profile(self._h, 0))
        return json.loads(self._lib.kipp_engine_profile_json(self._h).decode())

    def decode_burst(self, requests: list, tokens: list[int], steps: int) -> torch.Tensor:
        """Greedy decoding of ``steps`` tokens for every request without the host in
        the loop.  ``tokens[i]`` is the next token of ``requests[i]`` (its logits
        give the first new token).  Returns int32 ``[steps, len(requests)]`` (host
        memory): row k holds the tokens chosen at step k.  The step is captured in a
        CUDA graph together with its argmax, the hand-over of the chosen tokens and
        the move of every request to its next position, so a burst is a run of graph
        replays with no copy and no other launch in between.  Pages for all steps
        are taken first (``OutOfPages`` leaves every request as it was).  Callers
        that must look at every token (stop tokens, sampling with penalties) use
        :meth:`step`."""
        n = len(requests)
        out = torch.empty((max(steps, 0), n), dtype=torch.int32)
        if n == 0 or steps <= 0:
            return out
        if len(tokens) != n:
            raise ValueError("one next token per request")
        for r in requests:
            if not self.is_live(r):
                raise ValueError(f"decode_burst: request {r!r} is not live (feed its prompt with step())")
        rids = (ctypes.c_int64 * n)(*[self._id(r) for r in requests])
        toks = (ctypes.c_int32 * n)(*[int(t) for t in tokens])
        with torch.cuda.device(self.device):
            self._stream.wait_stream(torch.cuda.current_stream())
            self._check(self._lib.kipp_engine_decode_burst(self._h, rids, toks, n, int(steps), out.data_ptr()))
        return out

    def sample(self, params, rng_states: list[int], recent=None) -> list[int]:
        """One token for each row of the last step's logits (see
        ``sampling.Sampler``); ``rng_states`` is updated in place."""
        from ..sampling.params import to_native
        rows = len(params)
        if rows == 0:
            return []
        arr, keep = to_native(params, recent)
        states = (ctypes.c_uint64 * rows)(*[int(s) for s in rng_states])
        out = (ctypes.c_int32 * rows)()
        self._check(self._lib.kipp_engine_sample(self._h, arr, states, rows, out))
        for i in range(rows):
            rng_states[i] = int(states[i])
        del keep
        return list(out)

    def run_part(self, entries, run_index: int, which: str, input: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, output: Optional[torch.Tensor] = None) -> None:
        """One part of one run alone, on a step of its own (tests of the parts)."""
        entries, arr, keep = self._entries(entries)
        for t in (input, residual, output):
            if t is not None and (not t.is_cuda or not t.is_contiguous()):
                raise ValueError("run_part takes contiguous CUDA tensors")
        ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())   # noqa: E731
        with torch.cuda.device(self.device):
            self._stream.wait_stream(torch.cuda.current_stream())
            self._check(self._lib.kipp_engine_debug_part(self._h, arr, len(entries), run_index, which.encode(),
                                                         ptr(input), ptr(residual), ptr(output)))
            torch.cuda.current_stream().wait_stream(self._stream)
        del keep

    # -- accounting -----------------------------------------------------------------
    def info(self) -> dict:
        """What is loaded and what it may hold (the reference's kipp_model_info and
        kipp_session_info in one, src/kipp.h:109-145, 172-200)."""
        info = json.loads(self._lib.kipp_engine_info(self._h).decode())
        info["live_requests"] = {self._owners.obj_of(int(k)): v for k, v in info["live_requests"].items()}
        info["dtype"] = str(self.dtype)
        info["device"] = str(self.device)
        return info

    def _counter(self, name: str) -> int:
        return int(self.info()["counters"][name])

    def kernel_launches(self) -> int:
        """Kernels of this package run so far: launched directly or replayed in graphs."""
        return self._counter("kernel_launches")

    graph_replays = property(lambda self: self._counter("graph_replays"))
    steps_run = property(lambda self: self._counter("steps_run"))
    last_h2d_bytes = property(lambda self: self._counter("last_h2d_bytes"))
    last_forward_launches = property(lambda self: self._counter("last_forward_launches"))

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads (each weight once)."""
        return int(self.info()["weight_bytes"])

    def cache_bytes_per_token(self) -> int:
        return int(self.info()["cache_bytes_per_token"])
