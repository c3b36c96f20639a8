"""Beam search host logic on the CPU: the two-heap queue against its restatement and hand-worked cases, the placement of
surviving hypotheses on engine sequences, and the whole driver against the restated reference loop on a stand-in model
(GPT.cs:236-310, Decoder.cs:447-517, Utils/BeamSearch.cs, AdvUtils/FixedSizePriorityQueue.cs)."""
import numpy as np
import pytest

from oracle import beam_oracle
from seq2seqsharp_b200.beam import BestN, Hypothesis, beam_search, expand_and_select, place
from seq2seqsharp_b200.gpt import DecodingOptions, DecodingStrategyEnums as DS


def _kept(cap, scores):
    q = BestN(cap)
    for i, s in enumerate(scores):
        q.push(s, i)
    return [(float(s), v) for s, v in q.items()]


def test_queue_hand_worked_cases():
    # capacity 2: 3 goes to the upper heap, 1 enters the lower heap and is lifted across, 2 replaces the worst (3)
    assert _kept(2, [3.0, 1.0, 2.0]) == [(1.0, 1), (2.0, 2)]
    # capacity 1 keeps the best; an equal score does not replace it
    assert _kept(1, [2.0, 2.0, 1.5, 1.5]) == [(1.5, 2)]
    # an item that ties with the worst kept one is refused
    assert _kept(2, [1.0, 2.0, 2.0]) == [(1.0, 0), (2.0, 1)]
    # capacity 3 (upper heap of two cells, lower heap of one): 3 lands in the upper heap's second cell and is swapped with
    # the facing lower cell (2); descending input: 2 is lifted over 3, then 1 climbs to the root
    assert _kept(3, [1.0, 2.0, 3.0]) == [(1.0, 0), (2.0, 1), (3.0, 2)]
    assert _kept(3, [3.0, 2.0, 1.0]) == [(1.0, 2), (2.0, 1), (3.0, 0)]


@pytest.mark.parametrize("cap", [1, 2, 3, 4, 5, 6, 7, 8, 12])
def test_queue_matches_restatement(cap):
    rng = np.random.default_rng(100 + cap)
    for trial in range(300):
        n = int(rng.integers(1, 4 * cap + 3))
        # few distinct values: many ties
        scores = rng.choice(np.linspace(0.5, 3.0, int(rng.integers(2, 9))).astype(np.float32), size=n)
        if trial % 3 == 0:
            scores = rng.random(n).astype(np.float32)
        ref = beam_oracle.FixedSizePriorityQueue(cap, beam_oracle._compare_descending)
        for i, s in enumerate(scores):
            ref.Enqueue((np.float32(s), i))
        want = [(float(s), v) for s, v in ref]
        assert _kept(cap, scores) == want, (cap, list(scores))
        # whatever the order, the kept set is the `cap` smallest scores
        assert sorted(s for s, _ in want) == sorted(float(x) for x in np.sort(scores)[:cap])


def test_placement_keeps_first_child_and_fills_dropped_places():
    # item 0: pool 0, 2, 4; survivors: two children of 2 and one of 4 -> 2 and 4 stay, the second child of 2 goes to 0
    a = [Hypothesis([1], np.float32(1), parent=2), Hypothesis([2], np.float32(1), parent=4), Hypothesis([3], np.float32(1), parent=2)]
    # item 1: pool 1, 3, 5; all three from parent 1 (the step after the prefill)
    b = [Hypothesis([1], np.float32(1), parent=1), Hypothesis([2], np.float32(1), parent=1), Hypothesis([3], np.float32(1), parent=1)]
    copies = place([a, b], [[0, 2, 4], [1, 3, 5]])
    assert [h.slot for h in a] == [2, 4, 0] and [h.slot for h in b] == [1, 3, 5]
    assert copies == [(2, 0), (1, 3), (1, 5)]
    assert not {d for _, d in copies} & {s for s, _ in copies}


class _TableModel:
    """A stand-in language model: the distribution after a text is a fixed pseudo-random function of the whole text."""

    def __init__(self, V, seed, eos_boost=0.0):
        self.V, self.seed, self.eos_boost = V, seed, eos_boost

    def probs(self, ids):
        h = self.seed
        for t in ids:
            h = (h * 1000003 + int(t) + 1) % 2147483647
        rng = np.random.default_rng(h)
        x = rng.standard_normal(self.V).astype(np.float32) * 2.0
        x[0] += np.float32(self.eos_boost * len(ids))
        e = np.exp(x - x.max()).astype(np.float32)
        return (e / e.sum(dtype=np.float32)).astype(np.float32)


class _FakeOracle:
    def __init__(self, model):
        self.m = model

    def reset(self):
        pass

    def step(self, tokens, temperature, blocked):
        p = np.stack([self.m.probs(list(r)) for r in tokens])
        for b in blocked:
            p[:, b] += np.float32(-1.0)
        return None, p


class _FakeEngine:
    """Sequences with their own text, as the engine keeps caches: what the driver may rely on and nothing more."""

    def __init__(self, model, max_batch):
        self.m, self.max_batch, self.seqs = model, max_batch, []
        self.copies = 0

    def Reset(self):
        self.seqs = []

    def Batch(self):
        return len(self.seqs)

    def Prefill(self, prompts, opts):
        self.seqs = [[int(t) for t in r] for r in prompts]
        return np.zeros(len(self.seqs), dtype=np.int32)

    def BeamCandidates(self, K, opts):
        p = np.stack([self.m.probs(s) for s in self.seqs])
        for b in (opts.BlockedTokens or ()):
            p[:, b] += np.float32(-1.0)
        c = beam_oracle.candidates(p, K)
        ids = np.stack([i for i, _ in c], axis=1)
        lp = np.stack([l for _, l in c], axis=1)
        return ids, np.exp(lp), lp

    def BeamCopy(self, src, dst):
        assert not set(src) & set(dst) and len(set(dst)) == len(dst) and list(dst) == sorted(dst)
        for s, d in zip(src, dst):
            assert d <= len(self.seqs) and d < self.max_batch
            if d == len(self.seqs):
                self.seqs.append(None)
            self.seqs[d] = list(self.seqs[s])
            self.copies += 1

    def StepHost(self, last, opts):
        assert len(last) == len(self.seqs)
        for s, t in zip(self.seqs, last):
            s.append(int(t))
        return np.zeros(len(self.seqs), dtype=np.int32)


@pytest.mark.parametrize("K,B,eos_boost", [(1, 2, 0.0), (2, 1, 0.0), (3, 3, 0.0), (4, 2, 0.4), (5, 1, 0.9), (8, 2, 0.2)])
def test_driver_matches_restated_loop(K, B, eos_boost):
    model = _TableModel(V=23, seed=7 + K, eos_boost=eos_boost)
    rng = np.random.default_rng(K * 10 + B)
    prompts = rng.integers(1, 23, size=(B, 4)).astype(np.int32)
    opts = DecodingOptions(MaxTgtSentLength=14, BeamSearchSize=K, DecodingStrategy=DS.GreedySearch, BlockedTokens=[3] if K % 2 else None)
    steps_ref = []
    want_ids, want_scores = beam_oracle.beam_search(_FakeOracle(model), prompts, opts, record=lambda i, s: steps_ref.append(s))
    eng = _FakeEngine(model, max_batch=B * K)
    got = beam_search(eng, prompts, opts, trace=True)
    assert got.ids == want_ids
    np.testing.assert_array_equal(np.asarray(got.scores, dtype=np.float32), np.asarray(want_scores, dtype=np.float32))
    assert got.steps == len(steps_ref)
    for mine, ref in zip(got.trace, steps_ref):            # every step: same hypotheses in the same beam order
        assert [[(ids, np.float32(s)) for ids, s in item] for item in mine] == [[(ids, np.float32(s)) for s, ids in item] for item in ref]
    # the caches follow the hypotheses: every engine sequence holds its hypothesis' text but the newest id
    if got.steps > 1 and K > 1:
        assert eng.Batch() == B * K
    if K > 1 and eos_boost > 0.5:
        assert all(h[-1] == 0 for beam in got.ids for h in beam)      # ended by </s> everywhere, before the length limit
        assert got.steps < 10


def test_driver_refuses_what_it_does_not_offer():
    eng = _FakeEngine(_TableModel(11, 1), max_batch=2)
    with pytest.raises(ValueError):
        beam_search(eng, [[1, 2]], DecodingOptions(BeamSearchSize=3, MaxTgtSentLength=6))            # 3 beams need 3 sequences
    with pytest.raises(ValueError):
        beam_search(eng, [[1, 2]], DecodingOptions(BeamSearchSize=2, MaxTgtSentLength=6, DecodingStrategy=DS.Sampling))


def test_placement_invariants_on_random_survivor_sets():
    """Whatever the survivors' parents are: every hypothesis gets a sequence of its item's pool, no two share one, a copy's
    destination is never a sequence that still serves as a source, and a parent with at least one child keeps its rows."""
    rng = np.random.default_rng(77)
    for trial in range(400):
        K, B = int(rng.integers(1, 9)), int(rng.integers(1, 5))
        pools = [[b + k * B for k in range(K)] for b in range(B)]
        beams = []
        for b in range(B):
            n_parents = int(rng.integers(1, K + 1))
            parents = rng.choice(pools[b], size=n_parents, replace=False)
            beams.append([Hypothesis([0], np.float32(1), parent=int(rng.choice(parents))) for _ in range(K)])
        copies = place(beams, pools)
        dsts, srcs = [d for _, d in copies], [s for s, _ in copies]
        assert dsts == sorted(dsts) and len(set(dsts)) == len(dsts) and not set(dsts) & set(srcs)
        for b in range(B):
            slots = [h.slot for h in beams[b]]
            assert sorted(slots) == sorted(pools[b])                       # a permutation of the item's sequences
            used_parents = {h.parent for h in beams[b]}
            for p in used_parents:
                assert any(h.slot == p and h.parent == p for h in beams[b])   # its first child stays in place
            for h in beams[b]:
                assert h.slot == h.parent or (h.parent, h.slot) in copies
