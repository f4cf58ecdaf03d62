"""The generation loop: batches of unequal prompts, stop tokens, sequences that end earlier, and
as many batches one after another as there are requests.

Reference loop for one sequence (fastgguf.c:5284-5309): run the prompt, then repeat { sample; if
the token is a stop token, end WITHOUT emitting, feeding or recording it (:5296); emit; if the
context is full, end (:5300); run the token }.  ``max_tokens <= 0`` means until a stop token or a
full context (:5294).

Here a batch starts together: one step with all prompts (logits at each prompt's last token),
then one token per live sequence a step; a sequence that finishes leaves the step list and its
slot goes back when the batch ends, so the next batch uses it again.  The decisions live in
``run_batch`` over an abstract backend (acquire / release / step / sample / room), which the
tests drive with a fake on the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

from .batch import StepEntry


@dataclass
class Completion:
    prompt_len: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop" (a stop token was drawn) or "length" (max_tokens / context full)


def plan_batches(n_requests: int, batch_size: int) -> List[range]:
    """Requests are served in order, ``batch_size`` at a time."""
    if batch_size <= 0:
        raise ValueError("batch_size must be positive")
    return [range(b, min(n_requests, b + batch_size)) for b in range(0, n_requests, batch_size)]


def run_batch(backend, prompts: Sequence[Sequence[int]], first_index: int, max_tokens: int,
              stop_ids: Sequence[int], on_token=None) -> List[Completion]:
    """Generate for one batch of prompts that start together.  ``on_token(request_index, token)`` is called
    for every token as the host learns of it (the reference prints each token as it is made,
    fastgguf.c:5297-5298); stop tokens are not reported, as they are not emitted.

    backend.acquire(request_index, prompt) -> slot      backend.release(slot)
    backend.step(entries) -> logits handle              backend.sample(logits, slots) -> list of tokens
    backend.room(slot) -> tokens the slot can still take
    """
    stop = set(stop_ids)
    for p in prompts:
        if len(p) == 0:
            raise ValueError("a prompt needs at least one token")
    slots = [backend.acquire(first_index + i, p) for i, p in enumerate(prompts)]
    done = [Completion(len(p)) for p in prompts]
    try:
        live = list(range(len(prompts)))
        logits = backend.step([StepEntry(slots[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in live])
        while live:
            tokens = backend.sample(logits, [slots[i] for i in live])
            nxt = []
            for i, tok in zip(live, tokens):
                c = done[i]
                if tok in stop:                                   # not emitted, not fed, not recorded
                    c.finish_reason = "stop"
                    continue
                c.tokens.append(int(tok))
                if on_token is not None:
                    on_token(first_index + i, int(tok))
                if 0 < max_tokens <= len(c.tokens) or backend.room(slots[i]) <= 0:
                    c.finish_reason = "length"
                    continue
                nxt.append(i)
            live = nxt
            if live:
                logits = backend.step([StepEntry(slots[i], [done[i].tokens[-1]], [0]) for i in live])
    finally:
        for s in slots:
            backend.release(s)
    return done


def generate(engine, prompts: Sequence[Sequence[int]], params, *, max_tokens: int, stop_ids: Sequence[int],
             batch_size: int, on_token=None) -> List[Completion]:
    backend = engine.backend(params, stop_ids)
    out: List[Completion] = []
    for rng in plan_batches(len(prompts), batch_size):
        out.extend(backend.run_batch([prompts[i] for i in rng], rng.start, max_tokens, stop_ids, on_token))
    return out
