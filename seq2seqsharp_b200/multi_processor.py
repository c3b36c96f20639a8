"""Batch sharding of independent sequences over the GPUs of one box — the B200 form of the reference's
MultiProcessorNetworkWrapper + BaseSeq2SeqFramework.RunTest fan-out.

The reference keeps one replica of the network per device id inside one process
(Seq2SeqSharp/MultiProcessorNetworkWrapper.cs:20-294) and, at inference, cuts a batch into BatchSize / N contiguous
blocks, one per device, with the remainder run on device 0 afterwards, then merges the results in block order
(Seq2SeqSharp/Tools/BaseSeq2SeqFramework.cs:905-975).  Here every device is driven by its own process (rank) under
torch.distributed: each rank owns one engine replica, takes the same contiguous block, decodes it without any
collective on the data path, and the ids are gathered on the host.  A rank that fails reports the failure to every
other rank through the gather (nobody is left waiting on it).
"""
from dataclasses import replace
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np


def split_batch(batch_size: int, n_ranks: int) -> Tuple[List[Tuple[int, int]], Tuple[int, int]]:
    """(per-rank [begin, end) blocks, remainder block run on rank 0) — BaseSeq2SeqFramework.cs:908-909,944-946."""
    per = batch_size // n_ranks
    blocks = [(i * per, (i + 1) * per) for i in range(n_ranks)]
    return blocks, (n_ranks * per, batch_size)


class MultiProcessorNetworkWrapper:
    """One engine replica per rank; `RunTest` shards a batch of prompts and merges the generated ids in batch order."""

    def __init__(self, make_replica: Callable[[int], object], rank: int = 0, world_size: int = 1, group=None):
        self.rank, self.world_size, self.group = rank, world_size, group
        self.replica = make_replica(rank)          # GetNetworkOnDevice(deviceIdx) (GPT.cs:138-146)

    def _gather(self, payload):
        if self.world_size == 1:
            return [payload]
        import torch.distributed as dist
        out = [None] * self.world_size
        dist.all_gather_object(out, payload, group=self.group)
        return out

    def RunTest(self, tokens, decodingOptions, forward: Optional[Callable] = None):
        """tokens [B, S] on every rank (the reference reads the batch once and hands out ranges).  Returns the merged
        [B, n] ids on every rank.  `forward(replica, tokens_block, options)` defaults to RunForwardOnSingleDevice."""
        tokens = np.asarray(tokens, dtype=np.int32)
        B = tokens.shape[0]
        blocks, rem = split_batch(B, self.world_size)
        if forward is None:
            forward = lambda rep, t, o: rep.RunForwardOnSingleDevice(t, o, stop_on_eos=False)  # noqa: E731
        results, err = {}, None
        try:
            b, e = blocks[self.rank]
            if e > b:
                # each sequence keeps its own uniform stream wherever it runs: SeqBase = its index in the batch
                results[b] = np.asarray(forward(self.replica, tokens[b:e], replace(decodingOptions, SeqBase=decodingOptions.SeqBase + b)))
            if self.rank == 0 and rem[1] > rem[0]:
                results[rem[0]] = np.asarray(forward(self.replica, tokens[rem[0]:rem[1]],
                                                     replace(decodingOptions, SeqBase=decodingOptions.SeqBase + rem[0])))
        except Exception as ex:  # reported to all ranks below instead of leaving them in the gather
            err = "%s: %s" % (type(ex).__name__, ex)
        gathered = self._gather((err, results))
        failures = ["rank %d: %s" % (r, g[0]) for r, g in enumerate(gathered) if g[0] is not None]
        if failures:
            raise RuntimeError("RunTest failed on " + "; ".join(failures))
        merged = {}
        for _, res in gathered:
            merged.update(res)
        parts = [merged[k] for k in sorted(merged)]     # MergeResults: SortedDictionary by block id (BaseSeq2SeqFramework.cs:860-888)
        n = min(p.shape[1] for p in parts)
        return np.concatenate([p[:, :n] for p in parts], axis=0)


class RankLeft(RuntimeError):
    """Another rank of the job left (or stopped answering) between two steps."""

    def __init__(self, rank, reason):
        super().__init__("rank %d left the job: %s" % (rank, reason))
        self.rank, self.reason = rank, reason


class StepGuard:
    """Host-side liveness check between the steps of a multi-rank job whose kernels wait on each other (the
    tensor-parallel decode step exchanges partial sums inside one kernel per rank).  A rank may leave only between
    steps, with none of its kernels in flight; the others must learn of it on the host BEFORE their next launch,
    because a kernel that waits for a peer that will never arrive runs into its poll limit, and a peer that has freed
    its exchange memory must not be written to.  Each rank announces the step it is about to launch in a key-value
    store (any `torch.distributed` store), announces when it leaves, and checks the others before every launch.

    The reference has no counterpart: its devices are driven by threads of one process, and a failure of one device
    ends the whole call (Seq2SeqSharp/Tools/BaseSeq2SeqFramework.cs:905-963)."""

    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 5.0, poll_s: float = 0.01):
        self.store, self.rank, self.world, self.timeout_s, self.poll_s = store, rank, world_size, timeout_s, poll_s

    def announce(self, step: int):
        self.store.set("step/%d" % self.rank, str(int(step)))

    def leave(self, reason: str = "left"):
        self.store.set("left/%d" % self.rank, reason or "left")

    def check(self, step: int):
        """Returns once every other rank has announced `step` (or a later one); raises RankLeft when one of them has
        announced that it left, or has not announced the step within the timeout."""
        import time
        deadline = time.monotonic() + self.timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                if self.store.check(["left/%d" % r]):
                    raise RankLeft(r, self.store.get("left/%d" % r).decode("utf-8", "replace"))
                if self.store.check(["step/%d" % r]) and int(self.store.get("step/%d" % r)) >= step:
                    break
                if time.monotonic() > deadline:
                    raise RankLeft(r, "no announcement of step %d within %.1f s" % (step, self.timeout_s))
                time.sleep(self.poll_s)
