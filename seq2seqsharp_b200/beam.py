"""Beam search over the GPT token loop with one KV cache per hypothesis.

The reference (GPT.cs:236-304) keeps `beam2batchStatus`, a list per beam of one status (ids, score) per batch item; every
step it runs `GPTDecode` once per beam over the WHOLE text of its hypotheses (with more than one beam it uses no KV cache,
GPT.cs:242), takes BeamSearchSize candidates from each (first arg-max, zero it, again: Decoder.cs:447-517), adds
-log(p) to the hypothesis score (a new status starts at 1.0, Utils/BeamSearch.cs:31), and keeps per batch item the
BeamSearchSize candidates of smallest score through a fixed-size two-heap queue (`BeamSearch.GetTopNBSS`,
AdvUtils/FixedSizePriorityQueue.cs) whose enumeration order - not a sorted order - is the order of the beams from then on.
A hypothesis that has produced </s> is extended like any other; the loop ends when every hypothesis ends in </s> or at
MaxTgtSentLength.

Here every hypothesis is a sequence of the engine: the prompt is prefilled once per batch item, a surviving hypothesis
keeps its cache rows, further children of the same parent are copied over the rows of dropped hypotheses on the device
(`TSB200_GptBeamCopy`), and a step costs one forward of one token per hypothesis instead of the whole text.  Scores, the
queue and the order of the beams follow the reference to the letter so that outputs come in the same order.
"""
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np


class BestN:
    """At most `capacity` items, the ones with the smallest score, held the way the reference's queue holds them: an upper
    heap (best item at its root) and a lower heap (worst item at its root) of nearly equal size whose leaves face each
    other.  Only the order matters to a caller: `items()` walks the upper heap's array front to back, then the lower heap's
    back to front, exactly the enumeration of AdvUtils/FixedSizePriorityQueue.cs:308-314 with the descending comparer of
    Utils/BeamSearch.cs:38.  An item that ties with the worst kept one does not replace it."""

    def __init__(self, capacity: int):
        if capacity < 1:
            raise ValueError("capacity must be at least one")
        self.cap = capacity
        n_low = max(capacity // 2, 1)
        self.low: List[Optional[tuple]] = [None] * n_low                       # worst at [0]
        self.up: List[Optional[tuple]] = [None] * max(capacity - n_low, 1)     # best at [0]
        self.n = self.n_up = self.n_low = 0

    # "a should sit above b" in the upper heap (smaller score) / in the lower heap (larger score)
    @staticmethod
    def _wins(a, b, upper: bool) -> bool:
        d = np.float32(a[0]) - np.float32(b[0])
        return d < 0 if upper else d > 0

    def _sift_up(self, arr, i, upper):
        while i > 0:
            par = (i - 1) // 2
            if not self._wins(arr[i], arr[par], upper):
                break
            arr[i], arr[par] = arr[par], arr[i]
            i = par
        return i

    def _sift_down(self, arr, i, size, upper):
        while True:
            pick = i
            for ch in (2 * i + 1, 2 * i + 2):
                if ch < size and self._wins(arr[ch], arr[pick], upper):
                    pick = ch
            if pick == i:
                return i
            arr[i], arr[pick] = arr[pick], arr[i]
            i = pick

    # which upper-heap cells face lower-heap cell i
    def _facing_up(self, i):
        left = 2 * i + 1
        via_child = left if self.n_low <= left < self.n_up else i
        first = via_child
        second = i + 1 if (i == self.n_low - 1 and i % 2 == 1 and self.n_up > self.n_low) else via_child
        return first, second

    # which lower-heap cell faces upper-heap cell i (-1: none)
    def _facing_low(self, i):
        if i < self.n_low:
            return i
        return (i - 1) // 2 if i % 2 == 1 else i - 1

    def _lift_across(self, pos):
        """Lower-heap item at `pos` moves into the upper heap if it beats a facing cell; returns that cell or -1."""
        a, b = self._facing_up(pos)
        item = self.low[pos]
        to = -1
        if self._wins(item, self.up[a], True):
            to = a
        if self._wins(item, self.up[b], True) and (to == -1 or self._wins(self.up[a], self.up[b], True)):
            to = b
        if to >= 0:
            self.up[to], self.low[pos] = self.low[pos], self.up[to]
        return to

    def _drop_across(self, pos):
        """Upper-heap item at `pos` moves into the lower heap if the facing cell beats it; returns that cell or -1."""
        j = self._facing_low(pos)
        if j < 0 or j >= self.n_low or not self._wins(self.low[j], self.up[pos], True):
            return -1
        self.up[pos], self.low[j] = self.low[j], self.up[pos]
        return j

    def push(self, score, value) -> bool:
        item = (np.float32(score), value)
        if self.n == self.cap:
            if self.cap == 1:
                if not self._wins(item, self.up[0], True):
                    return False
                self.up[0] = item
                return True
            if not self._wins(item, self.low[0], True):
                return False
            self.low[0] = item
            at = self._sift_down(self.low, 0, self.n_low, False)
            if 2 * at + 2 < self.n_low:       # not on the boundary between the heaps
                return True
            moved = self._lift_across(at)
            if moved >= 0:
                self._sift_up(self.up, moved, True)
            return True
        self.n += 1
        if self.n_low < self.n_up:
            pos = self.n_low
            self.n_low += 1
            self.low[pos] = item
            moved = self._lift_across(pos)
            if moved < 0:
                self._sift_up(self.low, pos, False)
            else:
                self._sift_up(self.up, moved, True)
        else:
            pos = self.n_up
            self.n_up += 1
            self.up[pos] = item
            moved = self._drop_across(pos)
            if moved < 0:
                self._sift_up(self.up, pos, True)
            else:
                self._sift_up(self.low, moved, False)
        return True

    def items(self):
        return [self.up[i] for i in range(self.n_up)] + [self.low[i] for i in range(self.n_low - 1, -1, -1)]


@dataclass
class Hypothesis:
    ids: List[int]                 # prompt + generated ids
    score: np.float32              # 1.0 - sum of log probabilities (smaller is better)
    slot: int = -1                 # the engine sequence that holds its cache
    parent: int = -1               # slot of the hypothesis it extends (during selection)


@dataclass
class BeamResult:
    ids: List[List[List[int]]]     # [beam][batch item] generated ids (without the prompt)
    scores: List[List[float]]      # [beam][batch item]
    slots: List[List[int]] = field(default_factory=list)   # [beam][batch item] engine sequence holding the hypothesis' cache
    steps: int = 0
    copies: int = 0
    trace: list = field(default_factory=list)


def expand_and_select(beams: Sequence[Sequence[Hypothesis]], cand_ids, cand_logp, K: int) -> List[List[Hypothesis]]:
    """One selection round for every batch item: each hypothesis (in beam order) contributes its K candidates (in
    candidate order), the K of smallest score survive, in the queue's order.  cand_*[slot][j]."""
    out = []
    for hyps in beams:
        q = BestN(K)
        every = []
        for h in hyps:
            for j in range(K):
                # with one beam the reference does not score (outputSentScore false): the status keeps its initial 1.0
                score = np.float32(h.score + np.float32(-1.0) * np.float32(cand_logp[h.slot][j])) if K > 1 else np.float32(1.0)
                every.append(Hypothesis(ids=h.ids + [int(cand_ids[h.slot][j])], score=score, parent=h.slot))
        if K > 1:
            for c in every:
                q.push(c.score, c)
            out.append([v for _, v in q.items()])
        else:
            out.append(every)
    return out


def place(new_beams: List[List[Hypothesis]], pools: List[List[int]]):
    """Gives every surviving hypothesis a sequence of the engine: the first child of a parent stays in the parent's rows,
    every further child takes the rows of a hypothesis of the same batch item that was dropped (or that never existed yet).
    Returns the (source, destination) copies, destinations ascending."""
    copies = []
    for hyps, pool in zip(new_beams, pools):
        taken = set()
        for h in hyps:
            if h.parent not in taken:
                h.slot = h.parent
                taken.add(h.parent)
            else:
                h.slot = -1
        free = [s for s in pool if s not in taken]
        for h in hyps:
            if h.slot < 0:
                h.slot = free.pop(0)
                copies.append((h.parent, h.slot))
    copies.sort(key=lambda c: c[1])
    return copies


def beam_search(gpt, prompts, opts, trace: bool = False) -> BeamResult:
    """prompts [B, S] (equal lengths) -> the BeamSearchSize hypotheses of every batch item, beams in the reference's order.
    Greedy candidates only (the reference would draw Top-P samples per candidate with Sampling; not offered here)."""
    K = int(opts.BeamSearchSize)
    prompts = np.asarray(prompts, dtype=np.int32)
    if prompts.ndim != 2:
        raise ValueError("beam search takes prompts of equal length [batch, prompt_len]")
    if int(opts.DecodingStrategy) != 0:
        raise ValueError("beam search runs with DecodingStrategy GreedySearch")
    B, S = prompts.shape
    cfg = getattr(gpt, "cfg", None)
    if K > 1 and cfg is not None and int(cfg.pe) == 1 and cfg.ape_decode_pos0:
        # with a KV cache the reference adds position row 0 to every new token (Decoder.cs:674-677); with beams it has no cache,
        # re-runs whole texts and so adds each token's own row: an engine that mimics the cached quirk would not match it
        raise ValueError("beam search on a model with learned/sinusoid position rows needs an engine built with ape_decode_pos0=False")
    if B * K > gpt.max_batch:
        raise ValueError("beam search over %d prompts with %d beams needs max_batch >= %d" % (B, K, B * K))
    res = BeamResult(ids=[], scores=[])
    max_len = int(opts.MaxTgtSentLength)
    beams = [[Hypothesis(ids=[int(t) for t in prompts[b]], score=np.float32(1.0), slot=b)] for b in range(B)]
    pools = [[b + k * B for k in range(K)] for b in range(B)]
    if S < max_len:
        gpt.Reset()
        gpt.Prefill(prompts, opts)
    for i in range(S, max_len):
        cand_ids, _, cand_logp = gpt.BeamCandidates(K, opts)
        beams = expand_and_select(beams, cand_ids, cand_logp, K)
        copies = place(beams, pools)
        res.steps += 1
        if trace:
            res.trace.append([[(list(h.ids), float(h.score)) for h in hyps] for hyps in beams])
        if copies:    # also after the last selection: the engine's sequences then hold the final hypotheses (less their newest id)
            gpt.BeamCopy([c[0] for c in copies], [c[1] for c in copies])
            res.copies += len(copies)
        if all(h.ids[-1] == 0 for hyps in beams for h in hyps) or i + 1 >= max_len:
            break
        last = np.zeros(gpt.Batch(), dtype=np.int32)
        for hyps in beams:
            for h in hyps:
                last[h.slot] = h.ids[-1]
        gpt.StepHost(last, opts)
    n_beams = len(beams[0])
    res.ids = [[beams[b][k].ids[S:] for b in range(B)] for k in range(n_beams)]
    res.scores = [[float(beams[b][k].score) for b in range(B)] for k in range(n_beams)]
    res.slots = [[beams[b][k].slot for b in range(B)] for k in range(n_beams)]
    return res
