"""Host logic of the parked-cache pool (key rule, longest-head lookup, expiry, byte budget) with stand-in snapshots:
no GPU, no native call."""
import numpy as np
import pytest

from seq2seqsharp_b200.gpt import KvCachePool


class FakeSnap:
    def __init__(self, tokens, nbytes=100):
        self.tokens = np.asarray([tokens], dtype=np.int32)   # [1, T+1]: cached text + pending id
        self.B, self.T, self.nbytes = 1, len(tokens) - 1, nbytes
        self.closed = False

    def close(self):
        self.closed = True


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_key_drops_end_of_sentence_ids():
    # GenerateCacheKey removes "</s>" (id 0) from the text before joining it (GPT.cs:153-173)
    assert KvCachePool.key_of([5, 0, 7, 0]) == (5, 7)
    assert KvCachePool.key_of(np.array([[1, 2], [0, 3]])) == (1, 2, 3)


def test_longest_cached_head_wins_and_a_hit_leaves_the_pool():
    pool = KvCachePool(clock=Clock())
    a, b, c = FakeSnap([1, 2, 3, 9]), FakeSnap([1, 2, 3, 4, 5, 9]), FakeSnap([7, 7, 7])
    for s in (a, b, c):
        pool.put(s)
    assert len(pool) == 3
    assert pool.take([1, 2, 3, 4, 5, 6, 7]) is b        # 5 cached tokens beat 3
    assert len(pool) == 2                                # GPT.cs:245 removes the entry it picked up
    assert pool.take([1, 2, 3, 4, 5, 6, 7]) is a
    assert pool.take([1, 2, 3, 4, 5, 6, 7]) is None
    assert (pool.hits, pool.misses) == (2, 1)


def test_an_entry_must_leave_at_least_one_token_to_run():
    pool = KvCachePool(clock=Clock())
    pool.put(FakeSnap([1, 2, 3, 4]))                     # 3 cached tokens + pending id 4
    assert pool.take([1, 2, 3]) is None                  # nothing would be left to feed
    assert pool.take([1, 2, 8, 4]) is None               # differs inside the cached part
    s = pool.take([1, 2, 3, 5])                          # the pending id need not match: the request's text rules
    assert s is not None and s.T == 3


def test_entries_expire_after_the_time_to_live():
    clk = Clock()
    pool = KvCachePool(ttl_seconds=600.0, clock=clk)
    s = FakeSnap([1, 2, 3])
    pool.put(s)
    clk.t = 599.0
    assert len(pool) == 1
    clk.t = 601.0
    assert len(pool) == 0 and s.closed
    assert pool.take([1, 2, 3, 4]) is None


def test_byte_budget_evicts_the_entry_closest_to_expiry():
    clk = Clock()
    pool = KvCachePool(max_bytes=250, clock=clk)
    first, second, third = FakeSnap([1, 1, 1]), FakeSnap([2, 2, 2]), FakeSnap([3, 3, 3])
    pool.put(first)
    clk.t = 1.0
    pool.put(second)
    clk.t = 2.0
    pool.put(third)                                      # 300 bytes > 250: the oldest goes
    assert first.closed and not second.closed and not third.closed
    assert len(pool) == 2 and pool.nbytes == 200


def test_same_text_replaces_the_older_entry_and_batches_are_refused():
    pool = KvCachePool(clock=Clock())
    old, new = FakeSnap([4, 5, 6]), FakeSnap([4, 5, 6])
    pool.put(old)
    pool.put(new)
    assert old.closed and len(pool) == 1
    two = FakeSnap([1, 2, 3])
    two.B = 2
    with pytest.raises(ValueError):
        pool.put(two)
