"""The Python entry point: load a model folder, step it, generate from it.

``Engine`` wraps the host's engine (``fg_engine`` of ``csrc/fastgguf_engine.h``), which every program of the
framework drives - generation, the command line, trace replay, the benchmark and the tests share its model,
step function, cache and kernels; this class only marshals.  The option names of ``generate`` are the reference's
chat options with their meanings and defaults (``--temp 1.0`` 0 = greedy, ``--top-k 64`` 0 = off, ``--top-p 0.95``,
``--repeat-penalty 1.0`` 1 = off, ``--repeat-last-n 64``, ``--max-tokens 512`` 0 = until stop, ``--seed N``;
fastgguf.c:6957-6982), and ``ctx`` is its context length argument (default 2048, at least 64; :6972, :7085).
"""
from __future__ import annotations

import ctypes
import json
import os
from ctypes import byref, c_int, c_void_p
from typing import List, Optional, Sequence

from .. import capi
from ..config.base import ModelConfig
from ..registry import config_from_dir, spec_from_config
from ..sampling import SamplingParams
from ..weights import dtype_code, host_tensor_array
from .batch import StepEntry
from .generate import Completion, _token_callback, take_result
from .spec import ModelSpec

_DTYPE_NAMES = {capi.FG_F32: "float32", capi.FG_BF16: "bfloat16"}


def parse_dtype(name) -> str:
    """"bfloat16" or "float32" from a name or a torch dtype."""
    return _DTYPE_NAMES[dtype_code(name)]


class CacheView:
    """The engine's cache as tests and tools look at it."""

    def __init__(self, engine: "Engine"):
        self._e = engine

    def _info(self) -> dict:
        return self._e.info()

    @property
    def max_seq_len(self) -> int:
        return self._info()["max_seq_len"]

    @property
    def n_slots(self) -> int:
        return self._info()["slots"]

    @property
    def page_size(self) -> int:
        return self._info()["page_size"]

    @property
    def groups(self) -> list:
        return self._info()["groups"]

    def length(self, slot: int) -> int:
        out = c_int()
        capi.check(capi.lib().fg_slot_length(self._e._handle, int(slot), byref(out)))
        return out.value

    def free_pages(self, gi: int = 0) -> int:
        out = c_int()
        capi.check(capi.lib().fg_engine_free_pages(self._e._handle, int(gi), byref(out)))
        return out.value

    def live_slots(self) -> List[int]:
        live = []
        for s in range(self.n_slots):
            try:
                self.length(s)
                live.append(s)
            except capi.CacheError:
                pass
        return live

    def check(self) -> None:
        capi.check(capi.lib().fg_engine_cache_check(self._e._handle))


class DecodeSession:
    """One batch on the graph path, step by step (what the benchmark times): the prompts run and the first
    tokens are sampled at creation; ``advance(live)`` runs one recorded decode step."""

    def __init__(self, engine: "Engine", prompts, params: SamplingParams, stop_ids=()):
        self.engine, self.n = engine, len(prompts)
        flat, offs = capi.prompts_arrays(prompts)
        stops, n_stop = capi.int_array(stop_ids)
        s = params.to_struct()
        out = c_void_p()
        capi.check(capi.lib().fg_session_begin(engine._handle, self.n, flat, offs, byref(s), stops, n_stop, byref(out)))
        self._handle = out
        slots = (c_int * max(1, self.n))()
        capi.check(capi.lib().fg_session_slots(out, slots))
        self.slots = list(slots)[:self.n]
        self.launches_per_step = capi.lib().fg_session_launches_per_step(out)

    def advance(self, live: Sequence[int]) -> None:
        arr, n = capi.int_array(live)
        capi.check(capi.lib().fg_session_advance(self._handle, arr, n))

    def close(self) -> None:
        h, self._handle = self._handle, None
        if h:
            capi.lib().fg_session_close(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Engine:
    """A loaded model with its cache.  ``max_tokens`` sizes the cache: the most tokens that live sequences hold at
    any time, each sequence rounded up to a page of 64."""

    def __init__(self, config: Optional[ModelConfig] = None, *, model_dir: Optional[str] = None, tensors: Optional[dict] = None,
                 random_seed: Optional[int] = None, spec: Optional[ModelSpec] = None, dtype="bfloat16", max_tokens: int = 8192,
                 max_batch: int = 64, max_seq_len: Optional[int] = None, device="cuda:0", use_graphs: bool = True,
                 verbose: bool = False):
        self.config = config
        self.dtype = parse_dtype(dtype)
        self.max_batch, self.use_graphs = max_batch, use_graphs
        dev = str(device)
        opts = capi.EngineOptions()
        capi.lib().fg_engine_default_options(byref(opts))
        opts.dtype = dtype_code(dtype)
        opts.max_batch, opts.max_tokens, opts.max_seq_len = int(max_batch), int(max_tokens), int(max_seq_len or 0)
        opts.device = int(dev.split(":")[1]) if ":" in dev else 0
        opts.use_graphs, opts.verbose = int(bool(use_graphs)), int(bool(verbose))
        # the libraries the host opens by name are compiled here, on first use, for what this dtype needs
        capi.ensure_kernel_libraries(opts.dtype)
        out = c_void_p()
        l = capi.lib()
        if spec is not None:
            arr, n, keep = host_tensor_array(tensors or {})
            capi.check(l.fg_engine_create_from_spec(json.dumps(spec.to_json() if hasattr(spec, "to_json") else spec).encode("utf-8"),
                                                    arr, n, byref(opts), byref(out)))
        elif config is None:
            raise ValueError("an engine needs a configuration or a model spec")
        elif model_dir is not None:
            capi.check(l.fg_engine_create(config._handle, os.fspath(model_dir).encode("utf-8"), byref(opts), byref(out)))
        elif tensors is not None:
            arr, n, keep = host_tensor_array(tensors)
            capi.check(l.fg_engine_create_from_tensors(config._handle, arr, n, byref(opts), byref(out)))
        elif random_seed is not None:
            capi.check(l.fg_engine_create_random(config._handle, int(random_seed) & (2 ** 64 - 1), byref(opts), byref(out)))
        else:
            raise ValueError("an engine needs weights: a model folder, tensors, or a seed for random ones")
        self._handle = out
        self._info = None
        self.cache = CacheView(self)
        self.spec = spec if spec is not None else spec_from_config(config)

    def __del__(self):
        h, self._handle = getattr(self, "_handle", None), None
        if h:
            try:
                capi.lib().fg_engine_destroy(h)
            except Exception:
                pass

    @classmethod
    def from_dir(cls, model_dir: str, **kw) -> "Engine":
        """The model class is chosen by ``architectures[0]`` of ``model_dir/config.json``."""
        return cls(config_from_dir(model_dir), model_dir=model_dir, **kw)

    @classmethod
    def from_tensors(cls, config: ModelConfig, tensors: dict, **kw) -> "Engine":
        return cls(config, tensors=tensors, **kw)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, **kw) -> "Engine":
        """Random weights from the seeded generator, made on the device (the values ``write_random_model`` writes)."""
        return cls(config, random_seed=seed, **kw)

    @classmethod
    def from_spec(cls, spec, tensors: dict, **kw) -> "Engine":
        return cls(None, spec=spec, tensors=tensors, **kw)

    # ------------------------------------------------------------------ views
    def info(self) -> dict:
        if self._info is None:
            self._info = capi.take_json(capi.lib().fg_engine_info, self._handle)
        return self._info

    def expected_tensors(self) -> dict:
        return capi.take_json(capi.lib().fg_engine_expected_tensors, self._handle)

    @property
    def vocab_size(self) -> int:
        return self.info()["vocab_size"]

    @property
    def stream(self) -> int:
        """The CUDA stream the engine works on (a cudaStream_t as an integer)."""
        return capi.lib().fg_engine_stream(self._handle) or 0

    def stats(self) -> dict:
        return capi.take_json(capi.lib().fg_engine_stats, self._handle)

    def profile(self, on: bool = True) -> None:
        """Per-launcher device times: while on, kernels run one after another between two events each, and ``generate``
        runs its decode steps eagerly (sessions are refused)."""
        capi.check(capi.lib().fg_engine_profile(self._handle, 1 if on else 0))

    def profile_report(self) -> list:
        """``[{"name", "calls", "ms"}, ...]``, longest first, of everything launched since ``profile(True)`` or the last report."""
        return capi.take_json(capi.lib().fg_engine_profile_report, self._handle)

    def check_device(self) -> None:
        """Wait for the engine's stream; raise if a bounded wait inside a kernel ran out."""
        capi.check(capi.lib().fg_engine_check_device(self._handle))

    # ------------------------------------------------------------------ stepping
    def acquire(self) -> int:
        out = c_int()
        capi.check(capi.lib().fg_slot_acquire(self._handle, byref(out)))
        return out.value

    def release(self, slot: int) -> None:
        capi.check(capi.lib().fg_slot_release(self._handle, int(slot)))

    def _step(self, entries: Sequence[StepEntry], out_ptr_for) -> int:
        slots, n_seq = capi.int_array([e.slot for e in entries])
        n_tok, _ = capi.int_array([len(e.tokens) for e in entries])
        tokens, _ = capi.int_array([t for e in entries for t in e.tokens])
        want, at = [], 0
        for e in entries:
            for w in e.want:                         # places among the entry's own tokens -> rows of the step
                if not 0 <= int(w) < len(e.tokens):
                    raise capi.TokenError(f"slot {e.slot}: wanted place {w} is not among its {len(e.tokens)} tokens", capi.E_TOKEN)
                want.append(at + int(w))
            at += len(e.tokens)
        want_arr, n_want = capi.int_array(want)
        capi.check(capi.lib().fg_step(self._handle, n_seq, slots, n_tok, tokens, n_want, want_arr, out_ptr_for(n_want)))
        return n_want

    def step(self, entries: Sequence[StepEntry]):
        """Run the step; float32 logits ``[wanted, vocab]`` as a torch tensor on the device (None if none wanted)."""
        import torch
        holder = {}

        def out_ptr(n_want):
            if n_want == 0:
                return None
            holder["t"] = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device="cuda")
            torch.cuda.current_stream().synchronize()      # the buffer is free of work torch queued before
            return c_void_p(holder["t"].data_ptr())

        self._step(entries, out_ptr)
        return holder.get("t")

    def step_host(self, entries: Sequence[StepEntry]):
        """The same with the logits as a numpy array on the host (None if none wanted)."""
        import numpy as np
        holder = {}

        def out_ptr(n_want):
            if n_want == 0:
                return None
            holder["a"] = np.empty((n_want, self.vocab_size), dtype=np.float32)
            return c_void_p(holder["a"].ctypes.data)

        self._step(entries, out_ptr)
        return holder.get("a")

    def block_forward(self, schedule_entry: int, steps, x):
        """ONE schedule entry's block on rows ``x`` ([rows, hidden] float32 numpy, updated in place) through the real
        cache; ``steps`` is [(slot, rows of that sequence), ...].  For tests of a part alone."""
        slots, n = capi.int_array([s for s, _ in steps])
        n_tok, _ = capi.int_array([k for _, k in steps])
        capi.check(capi.lib().fg_engine_block_forward(self._handle, int(schedule_entry), n, slots, n_tok,
                                                      c_void_p(x.ctypes.data)))
        return x

    def session(self, prompts, params: Optional[SamplingParams] = None, stop_ids=()) -> DecodeSession:
        return DecodeSession(self, prompts, params or SamplingParams(temp=0.0), stop_ids)

    # ------------------------------------------------------------------ generation
    def generate(self, prompts: Sequence[Sequence[int]], *, temp: float = 1.0, top_k: int = 64, top_p: float = 0.95,
                 repeat_penalty: float = 1.0, repeat_last_n: int = 64, max_tokens: int = 512, seed: int = 0,
                 stop_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False, batch_size: Optional[int] = None,
                 on_token=None, use_graphs: Optional[bool] = None) -> List[Completion]:
        """Generate for every prompt (lists of token ids); returns one ``Completion`` per prompt.
        ``on_token(request_index, token)``, if given, is called for each generated token as the host sees it."""
        params = SamplingParams(temp=temp, top_k=top_k, top_p=top_p, repeat_penalty=repeat_penalty,
                                repeat_last_n=repeat_last_n, seed=seed)
        stops = () if ignore_eos else tuple(self.info()["stop_token_ids"] if stop_ids is None else stop_ids)
        flat, offs = capi.prompts_arrays(prompts)
        stop_arr, n_stop = capi.int_array(stops)
        s = params.to_struct()
        out = c_void_p()
        error = {}

        def reported(request, token):
            try:
                on_token(request, token)
            except BaseException as e:          # raised again once the host's loop has returned
                error.setdefault("e", e)

        cb = _token_callback(reported if on_token is not None else None)
        capi.check(capi.lib().fg_generate(self._handle, len(prompts), flat, offs, byref(s), int(max_tokens), stop_arr, n_stop,
                                          int(batch_size or 0), -1 if use_graphs is None else int(bool(use_graphs)), cb, None,
                                          byref(out)))
        done = take_result(out, prompts)
        if "e" in error:
            raise error["e"]
        return done
