"""Requests of different lengths through one engine: a fixed number of slots kept busy (continuous batching).

The reference serves one call of `GPT.RunForwardOnSingleDevice` at a time: it pads the prompts of the call to one length
(`BuildInTokens.PadSentences`, Decoder.cs:656), runs the token loop until every sequence has ended (GPT.cs:290-310), and
parks the call's K/V tensors in `MemoryCache.Default` under its text for the next call that starts with it
(GPT.cs:236-247, 312-328).  With a cache length, position, Philox step and stop flag per sequence (the engine's slot
operations) the same three things work per SEQUENCE: a request enters whichever slot is free - on top of a parked cache
that covers a head of its prompt, if the pool has one -, the token loop runs all occupied slots together, and a sequence
that ends is parked and makes room for the next request while the others run on.

Every request's tokens are the ones the same engine produces for that request alone: sequences do not see each other
(per-sequence lengths, row-independent kernels), and request i draws its Top-P uniforms from the Philox stream
(Seed, SeqBase + slot) with the slot's own step counter.
"""
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np


@dataclass
class Request:
    """One prompt and how many tokens to generate for it at most (generation also ends with </s> = id 0)."""
    rid: object
    tokens: List[int]
    max_new: int


@dataclass
class _Slot:
    req: Request
    out: List[int] = field(default_factory=list)


class ContinuousBatcher:
    """Drives an engine (`seq2seqsharp_b200.gpt.GPT` or anything with its slot methods) with up to `slots` sequences at a
    time.  `pool` (a `KvCachePool`) is optional: finished sequences are parked there and later requests that start with a
    parked text skip that part of their prompt."""

    def __init__(self, gpt, opts, slots: int, pool=None, max_tokens: Optional[int] = None, chunk: int = 8):
        self.gpt, self.opts, self.n_slots, self.pool = gpt, opts, int(slots), pool
        self.max_tokens = int(max_tokens if max_tokens is not None else opts.MaxTgtSentLength)
        self.chunk = max(1, int(chunk))
        self.stats = {"steps": 0, "admitted": 0, "pool_hits": 0, "tokens": 0, "slot_steps_idle": 0}

    # -- one request enters a slot: (parked head +) prompt -> first generated id
    def _admit(self, slot: int, req: Request) -> int:
        toks = [int(t) for t in req.tokens]
        if not toks:
            raise ValueError("request %r has an empty prompt" % (req.rid,))
        if len(toks) + 1 > self.max_tokens:
            raise ValueError("request %r: prompt of %d tokens does not fit the cache (%d)" % (req.rid, len(toks), self.max_tokens))
        snap = self.pool.take(toks) if self.pool is not None else None
        if snap is not None:
            self.gpt.SlotRestore(snap, slot)
            rest = toks[snap.T:]
            snap.close()
            self.stats["pool_hits"] += 1
        else:
            self.gpt.SlotReset(slot)
            rest = toks
        self.stats["admitted"] += 1
        return self.gpt.SlotExtend(slot, rest, self.opts)

    def _budget(self, s: _Slot) -> int:
        """Tokens the slot may still generate: the request's limit and the cache capacity."""
        cap = self.max_tokens - (len(s.req.tokens) + len(s.out))
        return min(s.req.max_new - len(s.out), cap)

    def run(self, requests) -> Dict[object, np.ndarray]:
        """Serves all requests; returns rid -> generated ids (without the prompt; a final </s> is kept)."""
        queue = deque(requests)
        slots: List[Optional[_Slot]] = [None] * self.n_slots
        done: Dict[object, np.ndarray] = {}
        self.gpt.Reset()
        self.gpt.SetPerSequenceState(True)

        def finish(i: int):
            s = slots[i]
            done[s.req.rid] = np.asarray(s.out, dtype=np.int32)
            self.stats["tokens"] += len(s.out)
            if self.pool is not None and s.out and s.out[-1] != 0:
                # park text + cache; a sequence that ended with </s> is parked without it by the pool's key rule anyway,
                # but its cache would end one position short of its text, so only open-ended sequences are kept
                self.pool.put(self.gpt.SlotSnapshot(i))
            slots[i] = None

        def fill(i: int):
            """Puts waiting requests into slot i until one of them needs the token loop (or the queue is empty)."""
            while queue:
                req = queue.popleft()
                if req.max_new <= 0:
                    done[req.rid] = np.zeros(0, dtype=np.int32)
                    continue
                first = self._admit(i, req)
                slots[i] = _Slot(req, [first])
                if first == 0 or self._budget(slots[i]) <= 0:
                    finish(i)
                    continue
                return
            if i < self.gpt.Batch():
                self.gpt.SlotReset(i)   # nothing waits: the slot stands still (pending </s>) while the others run on

        try:
            for i in range(self.n_slots):   # slots are claimed in order: index == number of sequences adds one
                if not queue:
                    break
                fill(i)
            while any(s is not None for s in slots):
                live = [s for s in slots if s is not None]
                k = max(1, min(self.chunk, min(self._budget(s) for s in live)))
                ids = self.gpt.Decode(k, self.opts, stop_on_eos=True)   # [batch, <= k]; ended sequences emit 0 and stand still
                self.stats["steps"] += ids.shape[1]
                self.stats["slot_steps_idle"] += ids.shape[1] * (self.gpt.Batch() - len(live))
                for i, s in enumerate(slots):
                    if s is None:
                        continue
                    ended = False
                    for t in ids[i]:
                        s.out.append(int(t))
                        if int(t) == 0:
                            ended = True
                            break
                    if ended or self._budget(s) <= 0:
                        finish(i)
                        fill(i)
        finally:
            self.gpt.SetPerSequenceState(False)
        return done
