"""Multi-rank host logic on CPU (gloo, world_size 2): batch sharding, merge order, per-sequence uniform streams, and
failure reporting when one rank raises.  No GPU involved: the replica is a stand-in with the engine's interface."""
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from seq2seqsharp_b200.gpt import DecodingOptions
from seq2seqsharp_b200.multi_processor import MultiProcessorNetworkWrapper, split_batch


def test_split_matches_reference_rule():
    assert split_batch(8, 2) == ([(0, 4), (4, 8)], (8, 8))
    assert split_batch(7, 2) == ([(0, 3), (3, 6)], (6, 7))          # remainder goes to device 0 afterwards
    assert split_batch(1, 4) == ([(0, 0)] * 4, (0, 1))
    assert split_batch(32, 8)[0][3] == (12, 16)


class FakeReplica:
    def __init__(self, rank, fail_on=None):
        self.rank, self.fail_on = rank, fail_on

    def RunForwardOnSingleDevice(self, tokens, opts, stop_on_eos=False):
        if self.fail_on == self.rank:
            raise MemoryError("OOM: KV-cache capacity exceeded")
        t = np.asarray(tokens)
        seq = opts.SeqBase + np.arange(t.shape[0])
        # "generated ids" depend on the prompt and on the sequence's own stream id, never on which rank ran it
        return np.stack([t.sum(1) + seq, t[:, 0] * 3 + seq, 100 * self.rank + 0 * seq], axis=1).astype(np.int32)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fail_on, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = MultiProcessorNetworkWrapper(lambda r: FakeReplica(r, fail_on), rank, world)
        tokens = np.arange(7 * 5, dtype=np.int32).reshape(7, 5)
        try:
            out = w.RunTest(tokens, DecodingOptions(SeqBase=10))
            q.put((rank, "ok", out.tolist()))
        except RuntimeError as ex:
            q.put((rank, "err", str(ex)))
    finally:
        dist.destroy_process_group()


def _run(fail_on):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, fail_on, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(res)


@pytest.mark.timeout(300)
def test_two_ranks_shard_and_merge_in_batch_order():
    res = _run(fail_on=None)
    tokens = np.arange(35, dtype=np.int32).reshape(7, 5)
    seq = 10 + np.arange(7)
    for rank, status, out in res:
        assert status == "ok"
        out = np.array(out)
        np.testing.assert_array_equal(out[:, 0], tokens.sum(1) + seq)       # batch order kept, per-sequence stream ids kept
        np.testing.assert_array_equal(out[:, 1], tokens[:, 0] * 3 + seq)
        np.testing.assert_array_equal(out[:, 2], [0, 0, 0, 100, 100, 100, 0])  # blocks 0-2 rank 0, 3-5 rank 1, remainder rank 0


@pytest.mark.timeout(300)
def test_a_failing_rank_is_reported_to_all_ranks():
    res = _run(fail_on=1)
    for rank, status, msg in res:
        assert status == "err" and "rank 1" in msg and "OOM" in msg
