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


# ---- tensor-parallel sharding rule (the one the engine applies) checked on CPU ranks with a gloo all-reduce -------------
def _tp_layer_partial(cfg, w, x, k=0):
    """One decoder layer on THIS rank's shard, numpy: returns the partial sums of the two row-parallel projections
    (before the all-reduce) so the caller can reduce them.  x [rows, d] is replicated.  Prefill of S = rows tokens, B = 1."""
    import math
    from oracle.np_oracle import act, layernorm, rmsnorm, rope, softmax
    f32 = np.float32
    a, f = "GPTDecoder.SelfAttn_%d" % k, "GPTDecoder.PosFFN_%d" % k

    def norm(v, prefix):
        g = w[prefix + ".m_alpha"].reshape(-1)
        return layernorm(v, g, w[prefix + ".m_beta"].reshape(-1), cfg.eps) if int(cfg.norm) == 0 else rmsnorm(v, g, cfg.eps)

    S, hd = x.shape[0], cfg.hd
    h = norm(x, a + ".layerNormQ")
    q = (h @ w[a + ".Q"] + w[a + ".Qb"]).reshape(S, -1, hd).transpose(1, 0, 2)
    kk = (h @ w[a + ".K"] + w[a + ".Kb"]).reshape(S, -1, hd).transpose(1, 0, 2)
    vv = (h @ w[a + ".V"] + w[a + ".Vb"]).reshape(S, -1, hd).transpose(1, 0, 2)
    pos = np.arange(S)
    q, kk = rope(q, pos, cfg.rope_base), rope(kk, pos, cfg.rope_base)
    grp = q.shape[0] // kk.shape[0]
    sc = (q @ np.repeat(kk, grp, 0).transpose(0, 2, 1)) * f32(1 / math.sqrt(hd))
    sc = sc + np.where(pos[None, :] <= pos[:, None], f32(0), f32(-30000.0))
    o = (softmax(sc.astype(f32)) @ np.repeat(vv, grp, 0)).transpose(1, 0, 2).reshape(S, -1)
    return (o @ w[a + ".W0"] + w[a + ".b0"]).astype(f32), h, f


def _tp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import dataclasses
        import torch
        from oracle.np_oracle import NpGPT, act
        from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, GPTConfig, MultiHeadAttentionTypeEnums as M, NormEnums as Nm,
                                           PositionEmbeddingEnums as P, synthetic_weights, tp_shard_weights)
        cfg = GPTConfig(L=1, d=64, H=4, Hkv=2, hd=16, F=96, V=53, norm=Nm.RMSNorm, act=A.SwiGLU, pe=P.RoPE, attn=M.GQA)
        w = synthetic_weights(cfg, 5, std=0.1, bias_std=0.05)
        ws = tp_shard_weights(cfg, w, rank, world)
        local = dataclasses.replace(cfg, H=cfg.H // world, Hkv=cfg.Hkv // world, F=cfg.F // world)
        rng = np.random.default_rng(0)
        x = rng.standard_normal((5, cfg.d)).astype(np.float32)

        def allreduce(v):
            t = torch.from_numpy(v.copy())
            dist.all_reduce(t)
            return t.numpy()

        part, _, f = _tp_layer_partial(local, ws, x)
        x1 = x + allreduce(part)                                   # one all-reduce after the out-projection
        from oracle.np_oracle import rmsnorm
        h2 = rmsnorm(x1, ws[f + ".layerNorm2.m_alpha"].reshape(-1), cfg.eps)
        u = act(3, (h2 @ ws[f + ".feedForwardLayer1.m_Whd"] + ws[f + ".feedForwardLayer1.m_Bd"]).astype(np.float32))
        u = u * (h2 @ ws[f + ".feedForwardLayer3.m_Whd"] + ws[f + ".feedForwardLayer3.m_Bd"])
        x2 = x1 + allreduce((u @ ws[f + ".feedForwardLayer2.m_Whd"] + ws[f + ".feedForwardLayer2.m_Bd"]).astype(np.float32))  # and one after the down-projection
        # unsharded reference on the same rank
        full, _, _ = _tp_layer_partial(cfg, w, x)
        y1 = x + full
        g2 = rmsnorm(y1, w[f + ".layerNorm2.m_alpha"].reshape(-1), cfg.eps)
        v = act(3, (g2 @ w[f + ".feedForwardLayer1.m_Whd"] + w[f + ".feedForwardLayer1.m_Bd"]).astype(np.float32))
        v = v * (g2 @ w[f + ".feedForwardLayer3.m_Whd"] + w[f + ".feedForwardLayer3.m_Bd"])
        y2 = y1 + (v @ w[f + ".feedForwardLayer2.m_Whd"] + w[f + ".feedForwardLayer2.m_Bd"])
        q.put((rank, float(np.abs(x2 - y2).max()), float(np.abs(y2).max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_tensor_parallel_sharding_rule_sums_to_the_unsharded_layer():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, scale in res:
        assert err <= 1e-5 * max(1.0, scale), "rank %d: sharded layer differs from the unsharded one by %g" % (rank, err)


# ---- a rank that leaves between steps is reported to the others before their next launch ---------------------------------
def _guard_worker(rank, world, port, mode, q):
    import datetime
    import time
    from seq2seqsharp_b200.multi_processor import RankLeft, StepGuard
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    guard = StepGuard(store, rank, world, timeout_s=2.0)
    done = 0
    try:
        for step in range(6):
            if rank == 1 and step == 3:
                if mode == "announced":
                    guard.leave("KV-cache capacity exceeded")   # leaves between steps, nothing of it in flight
                break                                           # mode "silent": just stops announcing
            guard.announce(step)
            guard.check(step)     # before the launch of `step`: everybody is still there
            done += 1             # (the launch itself)
        q.put((rank, "finished", done, ""))
    except RankLeft as ex:
        q.put((rank, "peer_left", done, str(ex)))
    if rank == 0:
        time.sleep(1.0)   # the store's server lives in rank 0: keep it up while rank 1 finishes


@pytest.mark.timeout(120)
@pytest.mark.parametrize("mode", ["announced", "silent"])
def test_a_rank_that_leaves_between_steps_is_seen_before_the_next_launch(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_guard_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict((r[0], r[1:]) for r in (q.get(timeout=60) for _ in procs))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert res[1][0] == "finished" and res[1][1] == 3
    status, done, msg = res[0]
    assert status == "peer_left" and done == 3 and "rank 1" in msg     # three steps ran, the fourth was never launched
    assert ("capacity" in msg) if mode == "announced" else ("no announcement of step 3" in msg)


# ---- teardown of peer-mapped memory: nobody frees before everybody has unmapped -------------------------------------------
def _teardown_worker(rank, world, port, q):
    import time
    import types
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import ctypes as C
        from seq2seqsharp_b200 import gpt as G
        log = []

        class FakeLib:
            def __getattr__(self, name):
                def call(*a):
                    log.append((name, time.monotonic()))
                    return 1
                return call
        G.N.lib = lambda: FakeLib()
        g = G.GPT.__new__(G.GPT)
        g._h, g._comm, g._peer_mapped, g._group = C.c_void_p(1), C.c_void_p(2), True, None
        if rank == 1:
            time.sleep(0.5)   # a late rank: the early one must wait for it before freeing
        g.close()
        q.put((rank, log))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_tensor_parallel_teardown_is_two_phase():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_teardown_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    for r in (0, 1):
        assert [n for n, _ in res[r]] == ["TSB200_GptTpClose", "TSB200_CommPeerClose", "TSB200_GptDestroy", "TSB200_CommDestroy"]
    last_unmap = max(t for r in (0, 1) for n, t in res[r] if n == "TSB200_CommPeerClose")
    first_free = min(t for r in (0, 1) for n, t in res[r] if n == "TSB200_GptDestroy")
    assert first_free >= last_unmap      # CLOCK_MONOTONIC is shared by the processes of one host
