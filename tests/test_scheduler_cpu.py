"""The slot scheduler's host logic against a fake engine (no GPU): every request must get exactly the tokens it gets
when it is generated alone, whatever shares the batch with it, with and without the cache pool."""
import numpy as np
import pytest

from seq2seqsharp_b200.gpt import DecodingOptions, KvCachePool
from seq2seqsharp_b200.scheduler import ContinuousBatcher, Request

V = 53


def next_id(text):
    """A deterministic 'model': the next id is a hash of the whole text; id 0 (</s>) comes up now and then."""
    h = 1469598103934665603
    for t in text:
        h = ((h ^ (t + 1)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return int((h >> 17) % V) if (h >> 11) % 9 else 0


def alone(prompt, max_new):
    text, out = list(prompt), []
    while len(out) < max_new:
        nid = next_id(text)
        out.append(nid)
        if nid == 0:
            break
        text.append(nid)
    return out


class FakeSnapshot:
    def __init__(self, text, pending):
        self.B, self.T = 1, len(text)
        self.tokens = np.asarray([list(text) + [pending]], dtype=np.int32)
        self.nbytes = 4 * (len(text) + 1)
        self.text, self.pending, self.closed = list(text), pending, False

    def close(self):
        self.closed = True


class FakeEngine:
    """The engine's slot semantics: a slot holds its cached text and a pending id; a decode step feeds the pending id,
    caches it and produces the next one; with the stop rule a slot whose pending id is </s> stands still."""

    def __init__(self, capacity):
        self.capacity, self.slots, self.per_seq = capacity, [], False
        self.calls = []

    def Reset(self):
        self.slots = []

    def SetPerSequenceState(self, on=True):
        self.per_seq = bool(on)

    def Batch(self):
        return len(self.slots)

    def _claim(self, slot):
        assert 0 <= slot <= len(self.slots) < self.capacity + 1 and slot < self.capacity
        if slot == len(self.slots):
            self.slots.append({"text": [], "pending": 0})

    def SlotReset(self, slot):
        self._claim(slot)
        self.slots[slot] = {"text": [], "pending": 0}

    def SlotSnapshot(self, slot):
        s = self.slots[slot]
        assert s["text"]
        return FakeSnapshot(s["text"], s["pending"])

    def SlotRestore(self, snap, slot):
        self._claim(slot)
        self.slots[slot] = {"text": list(snap.text), "pending": snap.pending}

    def SlotExtend(self, slot, tokens, opts):
        self._claim(slot)
        assert len(tokens) >= 1
        s = self.slots[slot]
        s["text"] = s["text"] + [int(t) for t in tokens]     # the pending id is overwritten by the caller's text
        s["pending"] = next_id(s["text"])
        self.calls.append(("extend", slot, len(tokens)))
        return s["pending"]

    def Decode(self, n, opts, stop_on_eos=False):
        assert self.per_seq and stop_on_eos and n >= 1
        out = []
        for _ in range(n):
            row = []
            for s in self.slots:
                if s["pending"] == 0:
                    row.append(0)
                    continue
                s["text"].append(s["pending"])
                s["pending"] = next_id(s["text"])
                row.append(s["pending"])
            out.append(row)
            if all(x == 0 for x in row):
                break
        return np.asarray(out, dtype=np.int32).T.reshape(len(self.slots), -1)


def _requests(rng, n):
    return [Request(i, [int(t) for t in rng.integers(1, V, size=int(rng.integers(1, 12)))], int(rng.integers(0, 15))) for i in range(n)]


@pytest.mark.parametrize("slots,chunk", [(1, 1), (3, 4), (4, 8), (8, 3)])
def test_every_request_gets_the_tokens_it_gets_alone(slots, chunk):
    rng = np.random.default_rng(slots * 10 + chunk)
    reqs = _requests(rng, 23)
    eng = FakeEngine(slots)
    opts = DecodingOptions(MaxTgtSentLength=64)
    b = ContinuousBatcher(eng, opts, slots=slots, max_tokens=64, chunk=chunk)
    got = b.run(reqs)
    assert set(got) == {r.rid for r in reqs}
    for r in reqs:
        assert list(got[r.rid]) == alone(r.tokens, r.max_new), r
    assert b.stats["admitted"] == sum(1 for r in reqs if r.max_new > 0)
    assert not eng.per_seq                     # switched off again


def test_cache_capacity_bounds_a_sequence():
    eng = FakeEngine(2)
    opts = DecodingOptions(MaxTgtSentLength=16)
    prompt = [3, 4, 5, 6, 7, 8, 9, 10, 11, 12]
    got = ContinuousBatcher(eng, opts, slots=2, max_tokens=16).run([Request("a", prompt, 100)])
    want = alone(prompt, 16 - len(prompt))     # prompt + generated tokens must fit the cache
    assert list(got["a"]) == want
    with pytest.raises(ValueError, match="does not fit"):
        ContinuousBatcher(eng, opts, slots=2, max_tokens=8).run([Request("b", prompt, 3)])
    with pytest.raises(ValueError, match="empty prompt"):
        ContinuousBatcher(eng, opts, slots=2, max_tokens=8).run([Request("c", [], 3)])


def test_parked_sequences_shorten_later_prompts():
    """A request that continues an earlier one (its prompt = that prompt + its answer + more text) finds the parked cache
    and runs only the new part of its prompt; its tokens are the same as without the pool."""
    eng = FakeEngine(2)
    opts = DecodingOptions(MaxTgtSentLength=128)
    pool = KvCachePool()
    first = Request("q1", [7, 8, 9, 10, 11], 6)
    out1 = alone(first.tokens, first.max_new)
    assert out1[-1] != 0, "pick a prompt whose answer is open-ended"
    follow = Request("q2", first.tokens + out1 + [21, 22, 23], 5)
    other = Request("q3", [31, 32], 4)
    b = ContinuousBatcher(eng, opts, slots=2, pool=pool, max_tokens=128)
    got = b.run([first, other])
    assert list(got["q1"]) == out1 and len(pool) >= 1
    eng.calls.clear()
    got = b.run([follow])
    assert list(got["q2"]) == alone(follow.tokens, follow.max_new)
    assert b.stats["pool_hits"] == 1
    # the parked cache held prompt + answer except the pending last token: the follow-up ran only the rest
    assert eng.calls[0] == ("extend", 0, len(follow.tokens) - (len(first.tokens) + len(out1) - 1))
