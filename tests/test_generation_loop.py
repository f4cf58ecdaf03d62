"""The generation loop's decisions - the host's ``run_batch`` and ``run_batch_late`` - driven by a fake backend on
the CPU through the C interface's callbacks."""
import pytest

from fastgguf_b200.engine.generate import plan_batches, run_batch, run_batch_late


class FakeBackend:
    """Sequences "generate" scripted tokens; records every step so that the test can check what was fed."""

    def __init__(self, scripts, capacity=1000, n_slots=4):
        self.scripts, self.capacity = scripts, capacity
        self.free = list(range(n_slots - 1, -1, -1))
        self.len, self.owner, self.cursor, self.steps, self.released = {}, {}, {}, [], []

    def acquire(self, request_index, prompt):
        s = self.free.pop()
        self.len[s], self.owner[s], self.cursor[s] = 0, request_index, 0
        return s

    def release(self, s):
        assert s in self.len, "released twice"
        del self.len[s]
        self.free.append(s)
        self.released.append(s)

    def room(self, s):
        return self.capacity - self.len[s]

    def step(self, entries):
        self.steps.append([(self.owner[e.slot], list(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            self.len[e.slot] += len(e.tokens)
        return [e.slot for e in entries]

    def sample(self, logits, slots):
        assert logits == list(slots)
        out = []
        for s in slots:
            out.append(self.scripts[self.owner[s]][self.cursor[s]])
            self.cursor[s] += 1
        return out


def test_plan_batches():
    assert [list(r) for r in plan_batches(7, 3)] == [[0, 1, 2], [3, 4, 5], [6]]
    assert plan_batches(0, 4) == []
    with pytest.raises(ValueError):
        plan_batches(3, 0)


def test_status_codes_of_the_c_interface():
    """Every exported function returns a status; the message of the last failure is kept for the caller."""
    import ctypes
    from fastgguf_b200 import capi
    l = capi.lib()
    out = ctypes.c_void_p()
    assert l.fg_config_from_json(None, ctypes.byref(out)) == capi.E_USAGE and b"null" in l.fg_last_error()
    assert l.fg_config_from_json(b"{nope", ctypes.byref(out)) == capi.E_CONFIG and b"not valid JSON" in l.fg_last_error()
    assert l.fg_config_from_json(b'{"architectures": ["Nope"]}', ctypes.byref(out)) == capi.E_CONFIG
    assert l.fg_cache_create(b"[]", 0, 64, 1, 64, ctypes.byref(out)) == capi.E_USAGE
    assert l.fg_cache_create(b'[{"entry": 0, "n_kv_heads": 1, "head_dim": 16}]', 64, 64, 1, 64, ctypes.byref(out)) == capi.OK
    slot, n = ctypes.c_int(), ctypes.c_int()
    assert l.fg_cache_acquire(out, ctypes.byref(slot)) == capi.OK and slot.value == 0
    assert l.fg_cache_acquire(out, ctypes.byref(slot)) == capi.E_CAPACITY and b"slots" in l.fg_last_error()
    assert l.fg_cache_length(out, 7, ctypes.byref(n)) == capi.E_CACHE
    one, many = (ctypes.c_int * 1)(0), (ctypes.c_int * 1)(500)
    assert l.fg_cache_reserve(out, 1, one, many) == capi.E_CAPACITY          # beyond the longest sequence
    assert l.fg_cache_check(out) == capi.OK
    l.fg_cache_destroy(out)
    assert l.fg_spec_tensors(b'{"hidden_size": 8}', ctypes.byref(out)) == capi.E_CONFIG
    assert l.fg_register_part(2, b"x", None) == capi.E_USAGE


def test_prompts_in_one_step_then_one_token_each():
    b = FakeBackend({0: [10, 11, 12], 1: [20, 21, 22]})
    out = run_batch(b, [[1, 2, 3], [4]], 0, max_tokens=3, stop_ids=())
    assert [c.tokens for c in out] == [[10, 11, 12], [20, 21, 22]]
    assert all(c.finish_reason == "length" for c in out)
    assert b.steps[0] == [(0, [1, 2, 3], [2]), (1, [4], [0])]          # logits at each prompt's last token
    assert b.steps[1] == [(0, [10], [0]), (1, [20], [0])]
    assert len(b.steps) == 3                                            # the last sampled token is not fed
    assert sorted(b.released) == [0, 1]


def test_stop_token_is_not_emitted_fed_or_recorded_and_the_rest_go_on():
    b = FakeBackend({0: [10, 99, 12], 1: [20, 21, 22, 23]})
    out = run_batch(b, [[1], [2]], 0, max_tokens=4, stop_ids=(99,))
    assert out[0].tokens == [10] and out[0].finish_reason == "stop"
    assert out[1].tokens == [20, 21, 22, 23] and out[1].finish_reason == "length"
    fed = [t for step in b.steps for (owner, toks, _) in step if owner == 0 for t in toks]
    assert 99 not in fed and fed == [1, 10]
    assert [len(s) for s in b.steps] == [2, 2, 1, 1]                    # the shorter request left the batch


def test_stop_at_the_first_sample_and_all_stopping_ends_the_batch():
    b = FakeBackend({0: [99], 1: [99]})
    out = run_batch(b, [[1, 2], [3]], 0, max_tokens=8, stop_ids=(99,))
    assert [c.tokens for c in out] == [[], []] and len(b.steps) == 1 and len(b.released) == 2


def test_full_context_ends_with_length():
    b = FakeBackend({0: list(range(100, 120))}, capacity=6)
    out = run_batch(b, [[1, 2, 3]], 0, max_tokens=0, stop_ids=())      # 0 = until stop or full
    assert out[0].tokens == [100, 101, 102, 103] and out[0].finish_reason == "length"
    assert b.len == {} and sum(len(t) for s in b.steps for (_, t, _) in s) == 6


def test_slots_come_back_when_a_step_fails():
    class Failing(FakeBackend):
        def step(self, entries):
            if len(self.steps) == 1:
                raise RuntimeError("boom")
            return super().step(entries)
    b = Failing({0: [1, 2], 1: [3, 4]})
    with pytest.raises(RuntimeError):
        run_batch(b, [[5], [6]], 0, max_tokens=4, stop_ids=())
    assert sorted(b.released) == [0, 1]


def test_empty_prompt_is_refused_before_anything_is_taken():
    b = FakeBackend({0: [1]})
    with pytest.raises(ValueError):
        run_batch(b, [[1], []], 0, max_tokens=2, stop_ids=())
    assert b.released == [] and len(b.free) == 4


def test_request_seeds_and_sampling_params():
    from fastgguf_b200.sampling import SamplingParams, request_seed, resolve_seed
    assert request_seed(7, 0) == 7 and request_seed(7, 1) != request_seed(7, 2) != 7
    assert all(request_seed(s, i) != 0 for s in (1, 7) for i in range(50))
    assert resolve_seed(5) == 5 and resolve_seed(0) != 0
    with pytest.raises(ValueError):
        SamplingParams(top_k=5000).validate()
    assert SamplingParams(temp=0).greedy and not SamplingParams().penalizes and SamplingParams(repeat_penalty=1.2).penalizes


class FakeSession:
    """The device of the graph path replaced by scripts: it goes on past a stop token, as the device does."""

    def __init__(self, scripts, prompts, first_index=0):
        self.scripts, self.n = scripts, len(prompts)
        self.idx = [first_index + i for i in range(self.n)]
        self.cursor = [1] * self.n
        self.first_tokens = [scripts[j][0] for j in self.idx]
        self.advanced, self.closed = [], 0

    def advance(self, live):
        self.advanced.append(list(live))
        toks = [0] * self.n
        for i in live:
            s = self.scripts[self.idx[i]]
            toks[i] = s[self.cursor[i]] if self.cursor[i] < len(s) else 0
            self.cursor[i] += 1
        return toks

    def close(self):
        self.closed += 1


def _graph_path(scripts, prompts, first_index, max_tokens, stop_ids, capacity=1000, on_token=None):
    """The graph path's host loop (tokens are seen one step late) with the device replaced by scripts."""
    session = FakeSession(scripts, prompts, first_index)
    out = run_batch_late(session, prompts, first_index, max_tokens, stop_ids, capacity, on_token)
    return out, session


@pytest.mark.parametrize("scripts,prompts,max_tokens,stop,capacity", [
    ({0: [10, 11, 12], 1: [20, 21, 22]}, [[1, 2, 3], [4]], 3, (), 1000),
    ({0: [10, 99, 12, 13, 14], 1: [20, 21, 22, 23, 24]}, [[1], [2]], 4, (99,), 1000),
    ({0: [99], 1: [99]}, [[1, 2], [3]], 8, (99,), 1000),
    ({0: [5, 6, 7, 8, 9, 10, 11], 1: [99, 1, 1, 1, 1, 1, 1], 2: [7, 7, 99, 3, 3, 3, 3]}, [[1] * 4, [2] * 2, [3]], 6, (99,), 1000),
    ({0: [1, 2, 3, 4, 5, 6, 7, 8], 1: [9, 9, 9, 9, 9, 9, 9, 9]}, [[1, 2, 3, 4, 5], [6]], 0, (), 8),     # the cache fills up
])
def test_graph_path_decides_as_the_plain_loop_does(scripts, prompts, max_tokens, stop, capacity):
    plain = run_batch(FakeBackend({k: list(v) + [0] * 8 for k, v in scripts.items()}, capacity=capacity), prompts, 0,
                      max_tokens=max_tokens, stop_ids=stop)
    seen = []
    out, log = _graph_path(scripts, prompts, 0, max_tokens, stop, capacity, on_token=lambda r, t: seen.append((r, t)))
    assert [(c.tokens, c.finish_reason) for c in out] == [(c.tokens, c.finish_reason) for c in plain]
    assert log.closed == 1
    # every token is reported once, in order, and stop tokens are not
    for i, c in enumerate(out):
        assert [t for r, t in seen if r == i] == c.tokens
    # a request is never stepped after the host knows that it ended, and at most once after it ended
    for i, c in enumerate(out):
        steps_taken = sum(1 for live in log.advanced if i in live)
        assert steps_taken <= len(c.tokens) + 1


def test_plain_loop_reports_tokens_with_request_indices():
    seen = []
    b = FakeBackend({4: [10, 99], 5: [20, 21]})
    run_batch(b, [[1], [2]], 4, max_tokens=2, stop_ids=(99,), on_token=lambda r, t: seen.append((r, t)))
    assert seen == [(4, 10), (5, 20), (5, 21)]
