"""DecoderModel: parts assembled from a :class:`ModelSpec`, and the ONE step function.

``step`` takes a batch of sequences, each with its next tokens (all prompts of a batch of
unequal lengths in one step, then one token each - or any other cut), runs exactly those
tokens as one batch from the cache that earlier steps left, and returns float32 logits at
the wanted places.  Generation, trace replay, the benchmark and the tests all call this
function; there is no second forward pass.

Reference: ``forward`` (one token, fastgguf.c:4648-4907) and ``forward_chunk`` /
``forward_batch`` (a prompt in chunks of 64 with logits for its last token only, :4943-5143),
both for one sequence at an explicit position.  Order of work per layer as there: norm,
q/k/v, rotary, cache write, attention, output projection + residual, norm, gate/up, SiLU-mul,
down + residual; then the final norm and the head on the wanted rows only (:5113-5117).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..cache.paged import PagedKVCache, StatePool
from ..parts import base as parts_base
from ..parts.base import LayerIO, Runtime, TensorSpec
from ..parts.embedding import LMHead, TokenEmbedding
from ..weights.loader import TensorSource, load_tensors
from .batch import Batch, StepEntry, build_batch, validate_entries
from .spec import ModelSpec, PartSpec


def _freeze(v):
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, (list, tuple)):
        return tuple(_freeze(x) for x in v)
    return v


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec, self.runtime = spec, runtime
        self._positions: Dict[tuple, parts_base.PositionEncoding] = {}
        self._bound: List[tuple] = []            # (part, {local name -> checkpoint name})
        self.embedding = TokenEmbedding(runtime, **spec.embedding.params)
        self._bound.append((self.embedding, spec.embedding.tensors))
        self.blocks = []
        for layer in spec.layers:
            mixer = self._build("mixer", layer.mixer)
            ffn = self._build("feed_forward", layer.feed_forward)
            n1 = self._build("norm", layer.mixer_norm)
            n2 = self._build("norm", layer.feed_forward_norm)
            self.blocks.append(parts_base.lookup("block", layer.block)(mixer, ffn, n1, n2))
        self.final_norm = self._build("norm", spec.final_norm)
        self.head = LMHead(runtime, **spec.head.params)
        self._bound.append((self.head, spec.head.tensors))
        self.cache: Optional[PagedKVCache] = None
        self.state: Optional[StatePool] = None
        self._io: List[LayerIO] = []

    # ------------------------------------------------------------------ building
    def _build(self, role: str, ps: PartSpec):
        params = dict(ps.params)
        for k, v in list(params.items()):
            if isinstance(v, PartSpec):          # a nested part: position encodings are shared
                key = (v.kind, _freeze(v.params))
                if key not in self._positions:
                    self._positions[key] = parts_base.lookup("position", v.kind)(self.runtime, **v.params)
                params[k] = self._positions[key]
        part = parts_base.lookup(role, ps.kind)(self.runtime, **params)
        self._bound.append((part, ps.tensors))
        return part

    def expected_tensors(self) -> Dict[str, TensorSpec]:
        """Checkpoint name -> spec, for every tensor the parts declare."""
        out: Dict[str, TensorSpec] = {}
        for part, names in self._bound:
            for local, tspec in part.tensor_specs().items():
                if local not in names:
                    raise KeyError(f"{type(part).__name__} declares tensor '{local}' but the architecture "
                                   f"gives no checkpoint name for it")
                ck = names[local]
                if ck in out and out[ck].shape != tspec.shape:
                    raise ValueError(f"tensor '{ck}' is used with shapes {out[ck].shape} and {tspec.shape}")
                out.setdefault(ck, tspec)
        return out

    def load_weights(self, source: TensorSource) -> None:
        tensors = load_tensors(source, self.expected_tensors(), self.runtime.dtype, self.runtime.device,
                               self.spec.ignored_tensors)
        for part, names in self._bound:
            part.load({local: tensors[names[local]] for local in part.tensor_specs()})

    # ------------------------------------------------------------------ cache
    def make_cache(self, *, max_tokens: int, n_slots: int, max_seq_len: Optional[int] = None,
                   page_size: int = 64) -> PagedKVCache:
        """Size the cache: ``max_tokens`` is the most tokens live sequences hold at any time
        (each sequence rounded up to a page)."""
        limit = self.spec.max_positions
        max_seq_len = min(limit, max_seq_len or limit, (max_tokens + page_size - 1) // page_size * page_size)
        cache_req, state_req = {}, {}
        for i, run in enumerate(self.spec.schedule):
            mixer = self.blocks[run.layer].mixer
            if run.cache_from is None and mixer.cache_request() is not None:
                cache_req[i] = mixer.cache_request()
            if mixer.state_request() is not None:
                state_req[i] = mixer.state_request()
        self.cache = PagedKVCache(cache_req, max_tokens=max_tokens, max_seq_len=max_seq_len, n_slots=n_slots,
                                  page_size=page_size, dtype=self.runtime.dtype, device=self.runtime.device)
        self.state = StatePool(state_req, n_slots, self.runtime.device)
        self._io = []
        for i, run in enumerate(self.spec.schedule):
            owner = i if run.cache_from is None else run.cache_from
            io = LayerIO(write_cache=run.cache_from is None, state=self.state.of(i))
            if owner in self.cache.group_of_entry:
                gi = self.cache.group_of_entry[owner]
                io.group = gi
                io.k_pool, io.v_pool = self.cache.groups[gi].k_pools[owner], self.cache.groups[gi].v_pools[owner]
            self._io.append(io)
        for pe in self._positions.values():
            pe.prepare(max_seq_len)
        return self.cache

    def acquire_slot(self) -> int:
        s = self.cache.acquire()
        self.state.reset(s)
        return s

    def release_slot(self, s: int) -> None:
        self.cache.release(s)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the step's tokens; return float32 logits ``[wanted, vocab]`` (None if none wanted)."""
        validate_entries(entries, self.spec.vocab_size)
        steps = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(steps)                      # all or nothing; raises before any launch
        batch = build_batch(entries, self.cache, self.runtime.device)
        logits = self.forward(batch)
        self.cache.commit(steps)
        return logits

    def forward(self, batch: Batch) -> Optional[torch.Tensor]:
        """The layers over a prepared batch (pages reserved, integers on the device)."""
        blocks = [self.blocks[run.layer] for run in self.spec.schedule]

        def entry_norm(block):
            # the norm a block starts with, if whoever writes the residual stream may start it
            ok = getattr(block.mixer, "supports_deferred_norm", False) and getattr(block.mixer_norm, "deferrable", False)
            return block.mixer_norm if ok and self.runtime.dtype == torch.bfloat16 else None

        first = entry_norm(blocks[0]) if blocks else None
        # the final norm can be started by the last block when the head takes every row as it is
        head_norm = None
        if (batch.want_all and self.runtime.dtype == torch.bfloat16 and getattr(self.final_norm, "deferrable", False)
                and getattr(self.head, "supports_deferred_norm", False)):
            head_norm = self.final_norm
        if first is not None:
            x, pending = self.embedding.forward(batch.tokens, emit_norm=first)
        else:
            x, pending = self.embedding.forward(batch.tokens), None      # [M, E] float32 residual stream
        for i, block in enumerate(blocks):
            nxt = entry_norm(blocks[i + 1]) if i + 1 < len(blocks) else head_norm
            pending = block.forward(x, batch, self._io[i], pending=pending, next_norm=nxt)
        if batch.want_rows is None:
            return None
        if head_norm is not None and pending is not None and blocks:
            return self.head.forward(pending)
        return self.head.forward(self.final_norm.forward(x, rows=batch.want_rows))
