"""The cache's bookkeeping on the host: no page or slot is lost, held twice or freed twice."""
import random

import pytest

from fastgguf_b200.cache import CacheError, CacheFull, CacheRequest, PagedKVCache, cache_bytes


def make(requests=None, **kw):
    requests = requests or {0: CacheRequest(2, 16), 1: CacheRequest(2, 16)}
    args = dict(max_tokens=640, max_seq_len=512, n_slots=4)
    args.update(kw)
    return PagedKVCache(requests, **args)


def test_groups_share_requests_and_have_storage_of_their_own():
    req = {0: CacheRequest(2, 16), 1: CacheRequest(2, 16, window=100), 2: CacheRequest(2, 16), 3: CacheRequest(1, 32)}
    c = PagedKVCache(req, max_tokens=256, max_seq_len=256, n_slots=2)
    assert len(c.groups) == 3 and c.groups[0]["entries"] == [0, 2] and c.group_of_entry == {0: 0, 1: 1, 2: 0, 3: 2}
    assert [g["pages"] for g in c.groups] == [4, 4, 4] and c.groups[1]["window"] == 100 and c.groups[0]["window"] is None
    # a pool per entry: [pages + the reserved page 0, KV heads, 64, head size], keys and values, 4 bytes each
    b = cache_bytes(req, 256, dtype="float32")
    assert b["bytes"] == 2 * 4 * 5 * 64 * (3 * 2 * 16 + 1 * 32) and b["pages"] == 4
    assert b["bytes_per_token"] == 2 * 4 * (3 * 2 * 16 + 1 * 32)


def test_cache_memory_of_the_benchmark_models():
    """Keys and values of one token over all layers, in bfloat16: 32 / 112 / 128 KiB for the 1B / 3B / 8B sizes."""
    for layers, kv, hd, kib in ((16, 8, 64, 32), (28, 8, 128, 112), (32, 8, 128, 128)):
        b = cache_bytes({i: CacheRequest(kv, hd) for i in range(layers)}, 4096)
        assert b["bytes_per_token"] == kib * 1024
        assert b["bytes"] == (4096 // 64 + 1) * 64 * kib * 1024


def test_pages_follow_lengths_and_come_back():
    c = make()
    a, b = c.acquire(), c.acquire()
    c.reserve([(a, 5), (b, 130)])
    assert c.free_pages() == 10 - 1 - 3
    c.commit([(a, 5), (b, 130)])
    assert c.length(a) == 5 and c.length(b) == 130
    c.reserve([(a, 59)]); c.commit([(a, 59)])                 # exactly fills the page: no new page
    assert c.free_pages() == 6
    c.reserve([(a, 1)]); c.commit([(a, 1)])                   # crosses into the second page
    assert c.free_pages() == 5 and c.length(a) == 65
    t = c.block_table(0, [a, b], 3)
    assert t.shape == (2, 3) and (t[0, :2] > 0).all() and t[0, 2] == 0 and (t[1] > 0).all()
    assert len(set(t[t > 0].tolist())) == 5 and 0 not in t[t > 0]      # page 0 is never handed out
    c.check()
    c.release(a)
    assert c.free_pages() == 7
    c.release(b)
    assert c.free_pages() == 10 and c.live_slots() == []
    c.check()


def test_errors_do_not_change_anything():
    c = make(max_tokens=128)
    a = c.acquire()
    with pytest.raises(CacheFull):
        c.reserve([(a, 200)])                                  # needs 4 pages, 2 exist
    assert c.free_pages() == 2 and c.length(a) == 0
    b = c.acquire()
    with pytest.raises(CacheFull):
        c.reserve([(a, 100), (b, 100)])                        # together too many: nothing is taken
    assert c.free_pages() == 2
    with pytest.raises(CacheError, match="twice in one step"):
        c.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError, match="at least one token"):
        c.reserve([(a, 0)])
    c.release(b)
    with pytest.raises(CacheError, match="released twice"):
        c.release(b)
    with pytest.raises(CacheError, match="not held"):
        c.length(b)
    with pytest.raises(CacheError, match="does not exist"):
        c.release(17)
    c.check()


def test_slots_run_out_and_are_reused():
    c = make(n_slots=2)
    a, b = c.acquire(), c.acquire()
    with pytest.raises(CacheFull, match="slots"):
        c.acquire()
    c.release(a)
    assert c.acquire() == a                                    # the freed slot is the next one handed out
    c.check()


def test_longest_sequence_limit():
    c = make(max_tokens=2048, max_seq_len=100)
    a = c.acquire()
    c.reserve([(a, 100)]); c.commit([(a, 100)])
    with pytest.raises(CacheFull, match="longest sequence"):
        c.reserve([(a, 1)])


def test_windowed_group_gives_pages_back():
    c = PagedKVCache({0: CacheRequest(1, 16), 1: CacheRequest(1, 16, window=70)}, max_tokens=2048, max_seq_len=2048,
                     n_slots=2)
    s = c.acquire()
    c.reserve([(s, 300)])
    assert c.free_pages(0) == 32 - 5 and c.free_pages(1) == 32 - 5     # a long prompt needs all its pages for the step
    c.commit([(s, 300)])
    assert c.free_pages(0) == 27 and c.free_pages(1) == 32 - 2         # positions 230.. live: pages 3 and 4
    for _ in range(200):
        c.reserve([(s, 1)]); c.commit([(s, 1)])
        c.check()
    assert c.free_pages(1) >= 32 - 3 and c.free_pages(0) == 32 - 8
    c.release(s)
    assert c.free_pages(0) == 32 and c.free_pages(1) == 32


def test_page_table_grows_beyond_its_first_width():
    c = make({0: CacheRequest(1, 16)}, max_tokens=64 * 200, max_seq_len=64 * 200, n_slots=1)
    s = c.acquire()
    c.reserve([(s, 64 * 150)]); c.commit([(s, 64 * 150)])
    t = c.block_table(0, [s], 150)
    assert (t > 0).all() and len(set(t[0].tolist())) == 150
    c.check()


def test_random_traffic_keeps_the_invariants():
    rnd = random.Random(3)
    c = make(max_tokens=64 * 12, n_slots=5)
    live = {}
    for _ in range(2000):
        op = rnd.random()
        if op < 0.25 and len(live) < 5:
            try:
                live[c.acquire()] = 0
            except CacheFull:
                pass
        elif op < 0.45 and live:
            s = rnd.choice(list(live))
            c.release(s); del live[s]
        elif live:
            picks = rnd.sample(list(live), rnd.randint(1, len(live)))
            steps = [(s, rnd.choice([1, 1, 1, 7, 64, 100])) for s in picks]
            try:
                c.reserve(steps)
            except CacheFull:
                continue
            c.commit(steps)
            for s, n in steps:
                live[s] += n
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.release(s)
    c.check()
    assert c.free_pages() == 12
