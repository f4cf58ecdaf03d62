"""Running a batch on the engine: the plain backend of the generation loop, and the graph-replayed
decode path that serving uses.

Plain path: ``run_batch`` of ``generate.py`` over ``acquire / release / step / sample / room`` -
one ``Engine.step`` and one device->host read of the sampled tokens per step.

Graph path (``use_graphs``): the decode step of a batch - the model's layers, the sampler and
the feedback of the sampled tokens into the next step's inputs - is captured once per batch
size as a CUDA graph over fixed buffers and replayed.  Tokens and positions stay on the
device; the host only reserves pages (its bookkeeping is deterministic), uploads page-table
rows when a sequence crosses a page, replays, and reads the sampled tokens one step late to
decide about stop tokens.  A sequence that drew a stop token is therefore fed for one more
step; that step's output for it is dropped and its slot is released with the batch.  Rows of
finished sequences and padding rows point at the reserved page 0 and the sampler's spare state
row, so they change nothing that is read.  The decisions are the ones ``run_batch`` makes; the
tests compare both paths token for token.
"""
from __future__ import annotations

from collections import deque
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..sampling import Sampler, SamplingParams, request_seed, resolve_seed
from .batch import Batch, StepEntry
from .generate import Completion, run_batch

BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    raise ValueError(f"a batch of {n} sequences exceeds the largest fixed-shape step ({BUCKETS[-1]})")


class DecodeGraph:
    """Fixed buffers and the captured decode step for ``width`` rows."""

    def __init__(self, engine, sampler: Sampler, width: int):
        model, cache, dev = engine.model, engine.cache, engine.device
        self.width, self.sampler = width, sampler
        self.table_width = (cache.max_seq_len + cache.page_size - 1) // cache.page_size
        n_groups = len(cache.groups)
        B = width
        pad = lambda n: (n + 3) // 4 * 4
        sizes = [B, B, B, B + 1, B, B, B] + [B * self.table_width] * n_groups
        offs = np.cumsum([0] + [pad(s) for s in sizes])
        self.ints = torch.zeros(int(offs[-1]), dtype=torch.int32, device=dev)
        v = lambda i: self.ints[int(offs[i]):int(offs[i]) + sizes[i]]
        self.tokens, self.positions, self.row_seq, self.cu_rows = v(0), v(1), v(2), v(3)
        self.rows, self.want, self.active = v(4), v(5), v(6)
        self.tables = [v(7 + g).view(B, self.table_width) for g in range(n_groups)]
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.row_seq.copy_(ar[:B]); self.cu_rows.copy_(ar); self.want.copy_(ar[:B])
        self.rows.fill_(sampler.spare_row)
        self.next_tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.batch = Batch(n_seq=B, n_rows=B, tokens=self.tokens, positions=self.positions, row_seq=self.row_seq,
                           cu_rows=self.cu_rows, seq_start=self.positions, slots=self.rows, want_rows=self.want,
                           block_tables=self.tables, n_want=B, max_new=1, max_len=cache.max_seq_len,
                           single_token=True, want_all=True)
        self.model = model
        from ..ops.lib import launches
        before = launches()
        self._run()                                   # warm-up outside capture: loads modules, sets attributes
        self.launches_per_step = launches() - before
        torch.cuda.synchronize()
        self.tokens.zero_(); self.positions.zero_()
        self.graph = torch.cuda.CUDAGraph()
        # Objects of earlier engines (graphs, pinned buffers, events) must not be finalised in the middle
        # of the capture: their CUDA calls are not allowed while a stream captures.
        import gc
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, capture_error_mode="relaxed"):
                self._run()
        finally:
            if was_enabled:
                gc.enable()

    def _run(self) -> None:
        logits = self.model.forward(self.batch)
        self.sampler.sample(logits, self.rows, out=self.next_tokens)
        ops.decode_advance(self.tokens, self.positions, self.next_tokens, self.active)

    def replay(self) -> None:
        self.graph.replay()


class EngineBackend:
    def __init__(self, engine, params: SamplingParams, stop_ids: Sequence[int], use_graphs: Optional[bool] = None):
        self.engine = engine
        self.params = params
        self.seed = resolve_seed(params.seed)
        self.sampler = Sampler(params, engine.cache.n_slots, stop_ids, engine.device)
        self.use_graphs = engine.use_graphs if use_graphs is None else use_graphs
        self._graphs: Dict[int, DecodeGraph] = {}
        self.stats = {"steps": 0, "h2d_bytes": 0, "d2h_bytes": 0}

    def reseed(self) -> None:
        """A new call with seed 0 draws a new seed from the clock."""
        self.seed = resolve_seed(self.params.seed)

    # ------------------------------------------------------------------ plain backend
    def acquire(self, request_index: int, prompt: Sequence[int]) -> int:
        slot = self.engine.acquire()
        self.sampler.begin(slot, request_seed(self.seed, request_index), prompt)
        return slot

    def release(self, slot: int) -> None:
        self.engine.release(slot)

    def room(self, slot: int) -> int:
        return self.engine.cache.max_seq_len - self.engine.cache.length(slot)

    def step(self, entries: Sequence[StepEntry]):
        self.stats["steps"] += 1
        self.stats["h2d_bytes"] += 4 * sum(len(e.tokens) for e in entries)
        return self.engine.step(entries)

    def sample(self, logits, slots: Sequence[int]) -> List[int]:
        rows = torch.tensor(list(slots), dtype=torch.int32, device=self.engine.device)
        toks = self.sampler.sample(logits, rows)
        self.stats["d2h_bytes"] += 4 * len(slots)
        host = toks.cpu().tolist()
        ops.raise_on_device_error("decode step")
        return host

    # ------------------------------------------------------------------ batches
    def run_batch(self, prompts, first_index: int, max_tokens: int, stop_ids: Sequence[int],
                  on_token=None) -> List[Completion]:
        if self.use_graphs and len(prompts) <= BUCKETS[-1]:
            return self._run_batch_graphs(prompts, first_index, max_tokens, stop_ids, on_token)
        return run_batch(self, prompts, first_index, max_tokens, stop_ids, on_token)

    def _graph(self, width: int) -> DecodeGraph:
        g = self._graphs.get(width)
        if g is None:
            g = self._graphs[width] = DecodeGraph(self.engine, self.sampler, width)
        return g

    def _run_batch_graphs(self, prompts, first_index, max_tokens, stop_ids, on_token=None) -> List[Completion]:
        cache = self.engine.cache
        stop = set(stop_ids)
        n = len(prompts)
        session = DecodeSession(self, prompts, first_index)
        done = [Completion(len(p)) for p in prompts]
        try:
            # sample k is produced by step k (k = 0: the prompt step); the host sees it one step late
            pending = deque([(list(range(n)), session.first_tokens, None)])
            known_done = [False] * n                   # decided from tokens the host has seen

            def settle(block: bool) -> None:
                while pending and (block or len(pending) > 1 or pending[0][2] is None):
                    who, toks, ev = pending.popleft()
                    if ev is not None:
                        ev.synchronize()
                        toks = toks.tolist()
                    for i in who:
                        if known_done[i]:
                            continue
                        tok, c = toks[i], done[i]
                        if tok in stop:                # not emitted, not fed on purpose, not recorded
                            c.finish_reason, known_done[i] = "stop", True
                            continue
                        c.tokens.append(int(tok))
                        if on_token is not None:
                            on_token(first_index + i, int(tok))
                        if 0 < max_tokens <= len(c.tokens) or len(prompts[i]) + len(c.tokens) - 1 >= cache.max_seq_len:
                            c.finish_reason, known_done[i] = "length", True

            step_no = 0
            while True:
                settle(block=False)
                step_no += 1
                # a sequence takes decode step s when it is not known to have ended, when sample s - 1
                # cannot have been its last by length, and when the cache has room for the token
                live = [i for i in range(n) if not known_done[i]
                        and (max_tokens <= 0 or step_no < max_tokens)
                        and len(prompts[i]) + step_no <= cache.max_seq_len]
                if not live:
                    break
                host, ev = session.advance(live)
                pending.append((live, host, ev))
            settle(block=True)
            ops.raise_on_device_error("batch")
        finally:
            session.close()
        return done


class DecodeSession:
    """One batch on the graph path: the prompt step, then ``advance(live)`` once per decode step."""

    def __init__(self, backend: EngineBackend, prompts, first_index: int = 0):
        self.backend, self.prompts = backend, prompts
        eng, dev = backend.engine, backend.engine.device
        for p in prompts:
            if len(p) == 0:
                raise ValueError("a prompt needs at least one token")
        n = self.n = len(prompts)
        g = self.graph = backend._graph(bucket_for(n))   # captured before slots are taken: its warm-up uses page 0
        self.slots = [backend.acquire(first_index + i, p) for i, p in enumerate(prompts)]
        try:
            logits = backend.step([StepEntry(self.slots[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in range(n)])
            rows = torch.tensor(self.slots, dtype=torch.int32, device=dev)
            first = backend.sampler.sample(logits, rows)
            g.tokens.zero_(); g.positions.zero_(); g.active.zero_()
            g.rows.fill_(backend.sampler.spare_row)
            for t in g.tables:
                t.zero_()
            g.tokens[:n] = first
            g.positions[:n] = torch.tensor([len(p) for p in prompts], dtype=torch.int32, device=dev)
            g.rows[:n] = rows
            g.active[:n] = 1
            self.widths = [0] * n                      # page-table entries of each row already uploaded
            self.first_tokens = first.cpu().tolist()
            ops.raise_on_device_error("prompt step")
            backend.stats["d2h_bytes"] += 4 * n
        except BaseException:
            self.close()
            raise

    def advance(self, live: Sequence[int]):
        """One decode step for the sequences ``live`` (indices into the batch).  Returns the pinned
        host tensor that receives the sampled tokens of all rows and the event that says when."""
        backend, g = self.backend, self.graph
        cache, dev = backend.engine.cache, backend.engine.device
        steps = [(self.slots[i], 1) for i in live]
        cache.reserve(steps)
        live_set = set(live)
        for i in range(self.n):
            if i not in live_set and self.widths[i] >= 0:     # finished: page 0, spare sampler row, position 0
                for t in g.tables:
                    t[i].zero_()
                g.active[i] = 0
                g.positions[i] = 0
                g.rows[i] = backend.sampler.spare_row
                self.widths[i] = -1
        for i in live:                                 # upload page-table entries the step will touch
            need = (cache.length(self.slots[i]) + 1 + cache.page_size - 1) // cache.page_size
            if need > self.widths[i]:
                for gi, t in enumerate(g.tables):
                    row = cache.tables[gi][self.slots[i], self.widths[i]:need]
                    t[i, self.widths[i]:need].copy_(torch.from_numpy(row.copy()).pin_memory(), non_blocking=True)
                    backend.stats["h2d_bytes"] += 4 * (need - self.widths[i])
                self.widths[i] = need
        g.replay()
        cache.commit(steps)
        backend.stats["steps"] += 1
        host = torch.empty(g.width, dtype=torch.int32, pin_memory=True)
        host.copy_(g.next_tokens, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        backend.stats["d2h_bytes"] += 4 * g.width
        return host, ev

    def close(self) -> None:
        for s in self.slots:
            self.backend.release(s)
        self.slots = []
