"""The generation loop as Python reaches it: ``Completion`` records, and the loop's decisions over a backend
given as Python callables (what the host-side tests drive with a fake on the CPU).

The loop itself is the host's (``run_batch`` and ``run_batch_late`` in ``csrc/host/runner.cpp``).  Reference loop
for one sequence (fastgguf.c:5284-5309): run the prompt, then repeat { sample; if the token is a stop token, end
WITHOUT emitting, feeding or recording it (:5296); emit; if the context is full, end (:5300); run the token }.
``max_tokens <= 0`` means until a stop token or a full context (:5294).
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_void_p
from dataclasses import dataclass, field
from typing import List, Sequence

from .. import capi
from .batch import StepEntry

_REASONS = {0: "", 1: "stop", 2: "length"}


@dataclass
class Completion:
    prompt_len: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop" (a stop token was drawn) or "length" (max_tokens / context full)


def take_result(handle: c_void_p, prompts) -> List[Completion]:
    """The completions of an fg_result, which is destroyed."""
    l = capi.lib()
    try:
        out = []
        for i in range(l.fg_result_count(handle)):
            toks, n, why = ctypes.POINTER(c_int)(), c_int(), c_int()
            capi.check(l.fg_result_get(handle, i, byref(toks), byref(n), byref(why)))
            out.append(Completion(len(prompts[i]), [toks[k] for k in range(n.value)], _REASONS.get(why.value, "")))
        return out
    finally:
        l.fg_result_destroy(handle)


def plan_batches(n_requests: int, batch_size: int) -> List[range]:
    """Requests are served in order, ``batch_size`` at a time."""
    return [range(a, b) for a, b in capi.take_json(capi.lib().fg_plan_batches, int(n_requests), int(batch_size))]


def _token_callback(on_token):
    if on_token is None:
        return capi.TOKEN_CALLBACK(0)
    return capi.TOKEN_CALLBACK(lambda _user, request, token: on_token(request, token))


def run_batch(backend, prompts: Sequence[Sequence[int]], first_index: int, max_tokens: int,
              stop_ids: Sequence[int], on_token=None) -> List[Completion]:
    """The host's loop for one batch of prompts that start together, over a Python backend:

    backend.acquire(request_index, prompt) -> slot      backend.release(slot)
    backend.step(entries) -> logits handle              backend.sample(logits, slots) -> list of tokens
    backend.room(slot) -> tokens the slot can still take

    ``on_token(request_index, token)`` is called for every token as the host learns of it; stop tokens are not
    reported, as they are not emitted.  An exception raised by the backend ends the loop and is raised again
    after the slots went back."""
    state = {"logits": None, "error": None}

    def guard(fn):
        def wrapped(*args):
            try:
                return fn(*args) or 0
            except BaseException as e:          # carried over the C frames, raised again below
                state["error"] = e
                return capi.E_INTERNAL
        return wrapped

    def acquire(_u, index, prompt, n, slot_out):
        slot_out[0] = backend.acquire(index, [prompt[i] for i in range(n)])

    def step(_u, n_seq, slots, n_tok, tokens):
        entries, at = [], 0
        for i in range(n_seq):
            entries.append(StepEntry(slots[i], [tokens[at + k] for k in range(n_tok[i])], [n_tok[i] - 1]))
            at += n_tok[i]
        state["logits"] = backend.step(entries)

    def sample(_u, n, slots, out):
        toks = backend.sample(state["logits"], [slots[i] for i in range(n)])
        for i in range(n):
            out[i] = int(toks[i])

    def room(_u, slot, out):
        out[0] = int(backend.room(slot))

    cb = capi.LoopBackend(None, capi.ACQUIRE_FN(guard(acquire)), capi.RELEASE_FN(guard(lambda _u, s: backend.release(s))),
                          capi.STEP_FN(guard(step)), capi.SAMPLE_FN(guard(sample)), capi.ROOM_FN(guard(room)))
    flat, offs = capi.prompts_arrays(prompts)
    stops, n_stop = capi.int_array(stop_ids)
    out = c_void_p()
    code = capi.lib().fg_run_batch(byref(cb), len(prompts), flat, offs, int(first_index), int(max_tokens), stops, n_stop,
                                   _token_callback(on_token), None, byref(out))
    if state["error"] is not None:
        raise state["error"]
    capi.check(code)
    return take_result(out, prompts)


def run_batch_late(session, prompts: Sequence[Sequence[int]], first_index: int, max_tokens: int, stop_ids: Sequence[int],
                   max_seq_len: int, on_token=None) -> List[Completion]:
    """The graph path's host loop (sampled tokens reach the host one step late) over a Python session:
    ``session.first_tokens`` (list), ``session.advance(live) -> tokens of all rows``, ``session.close()``."""
    state = {"error": None}
    n = len(prompts)

    def begin(_u, count, first_out):
        try:
            for i in range(count):
                first_out[i] = int(session.first_tokens[i])
            return 0
        except BaseException as e:
            state["error"] = e
            return capi.E_INTERNAL

    def advance(_u, n_live, live, out):
        try:
            toks = session.advance([live[i] for i in range(n_live)])
            for i in range(n):
                out[i] = int(toks[i])
            return 0
        except BaseException as e:
            state["error"] = e
            return capi.E_INTERNAL

    def close(_u):
        session.close()
        return 0

    cb = capi.LateBackend(None, capi.BEGIN_FN(begin), capi.ADVANCE_FN(advance), capi.CLOSE_FN(close))
    flat, offs = capi.prompts_arrays(prompts)
    stops, n_stop = capi.int_array(stop_ids)
    out = c_void_p()
    code = capi.lib().fg_run_batch_late(byref(cb), n, flat, offs, int(first_index), int(max_tokens), stops, n_stop,
                                        int(max_seq_len), _token_callback(on_token), None, byref(out))
    if state["error"] is not None:
        raise state["error"]
    capi.check(code)
    return take_result(out, prompts)
