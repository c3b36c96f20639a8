"""Tensor-parallel engine on 2 GPUs (one process per GPU) against the CPU oracle and against the unsharded engine.
The fp16 config decodes through the persistent kernel with the exchange over peer memory inside it, the fp32 config
through per-operation launches with the peer-memory all-reduce; prefill-sized messages go through NCCL in both.
A second test runs ONE sequence, which the owner-partitioned persistent kernel serves (its partial sums cross the ranks
as 64-bit integer atomics into every rank's residual buffer), next to the stream-K kernel on the same weights.
Needs two visible GPUs; skipped otherwise.

Every generated step is checked: logits within the dtype's tolerance of the oracle's (1e-3 fp32, 2e-2 fp16, relative to
the largest |logit| of the step), ids by the recorded-tie rule of tests/test_gpt_gpu.py (an id may differ from the
oracle's only where the oracle's top-2 probabilities are closer than the tolerance; the comparison of that sequence
stops there), and the sharded engine's logits against the one-GPU engine's on the same weights."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _configs():
    from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, GPTConfig, MultiHeadAttentionTypeEnums as M, NormEnums as Nm,
                                       PositionEmbeddingEnums as P)
    return [GPTConfig(name="gqa", L=2, d=256, H=8, Hkv=4, hd=32, F=512, V=1999, norm=Nm.RMSNorm, act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16"),
            GPTConfig(name="mha", L=2, d=128, H=4, hd=32, F=256, V=997, norm=Nm.LayerNorm, act=A.ReLU, pe=P.RoPE, attn=M.MHA, dtype="float32")]


S_PROMPT, N_NEW = 20, 12


def _options(strat):
    from seq2seqsharp_b200.gpt import DecodingOptions
    return DecodingOptions(MaxTgtSentLength=S_PROMPT + N_NEW, DecodingStrategy=strat, TopP=0.9, BlockedTokens=[0], Seed=11)


def _step_by_step(gpt, prompt, opts):
    """Prefill + one Decode(1) per token so that every step's logits can be read back."""
    gpt.Reset()
    ids = np.zeros((prompt.shape[0], N_NEW), dtype=np.int32)
    logits = []
    ids[:, 0] = gpt.Prefill(prompt, opts)
    logits.append(gpt.Logits())
    for i in range(1, N_NEW):
        ids[:, i] = gpt.Decode(1, opts)[:, 0]
        logits.append(gpt.Logits())
    return ids, logits


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from seq2seqsharp_b200.gpt import DecodingOptions, DecodingStrategyEnums as DS, GPT, synthetic_weights
    from seq2seqsharp_b200.synthetic import prompt_ids
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out = {}
        for cfg in _configs():
            w = synthetic_weights(cfg, 7, std=0.05, bias_std=0.02)
            prompt = prompt_ids(3, 2, S_PROMPT, cfg.V)     # rows = 40 -> tensor-core GEMM in prefill for fp16
            for strat in (DS.GreedySearch, DS.Sampling):
                opts = _options(strat)
                gpt = GPT(cfg, device_id=rank, max_batch=2, max_tokens=40, tp_rank=rank, tp_size=world)
                gpt.LoadWeights(w)
                gpt.InitComm()
                out[(cfg.name, int(strat))] = _step_by_step(gpt, prompt, opts)
                # and the graph-replayed loop (ids fed back on the device) gives the same ids
                out[(cfg.name, int(strat), "loop")] = gpt.RunForwardOnSingleDevice(prompt, opts, stop_on_eos=False)
                gpt.close()
                if rank == 0:  # the same model on one GPU
                    one = GPT(cfg, device_id=0, max_batch=2, max_tokens=40)
                    one.LoadWeights(w)
                    out[(cfg.name, int(strat), "one_gpu")] = _step_by_step(one, prompt, opts)
                    one.close()
            gpt = GPT(cfg, device_id=rank, max_batch=2, max_tokens=40, tp_rank=rank, tp_size=world)
            gpt.FillSynthetic(7, 0.05, 0.02)        # device-side generation keeps only this rank's share as well
            gpt.InitComm()
            opts = DecodingOptions(MaxTgtSentLength=S_PROMPT + N_NEW, BlockedTokens=[0])
            out[(cfg.name, "fill")] = gpt.RunForwardOnSingleDevice(prompt, opts, stop_on_eos=False)
            gpt.close()
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(900)
def test_tensor_parallel_two_gpus_matches_oracle(native, oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from seq2seqsharp_b200.gpt import DecodingStrategyEnums as DS, synthetic_weights
    from seq2seqsharp_b200.synthetic import prompt_ids
    from tests.test_gpt_gpu import compare_run, rel_err, tol_for
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=800) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for cfg in _configs():
        w = synthetic_weights(cfg, 7, std=0.05, bias_std=0.02)
        prompt = prompt_ids(3, 2, S_PROMPT, cfg.V)
        tol = tol_for(cfg)
        for strat in (DS.GreedySearch, DS.Sampling):
            opts = _options(strat)
            key = (cfg.name, int(strat))
            d_ids, d_logits = res[0][key]
            # both ranks hold identical results: the exchange gives every rank the same bits
            np.testing.assert_array_equal(d_ids, res[1][key][0])
            for (la, _), (lb, _) in zip(d_logits, res[1][key][1]):
                np.testing.assert_array_equal(la, lb)
            np.testing.assert_array_equal(res[0][key + ("loop",)], d_ids)
            # against the oracle: logits at every step, ids by the recorded-tie rule
            orc = oracle.OracleGPT(cfg, w)
            steps = {}
            o_ids = orc.generate(prompt, opts, uniforms=lambda st, b: oracle.philox_uniform(opts.Seed, opts.SeqBase + b, st),
                                 stop_on_eos=False, record=lambda st, lg, p, n: steps.update({st: (lg.copy(), p.copy(), n.copy())}))
            ties = compare_run(oracle, cfg, o_ids, steps, d_ids, d_logits, opts, prompt)
            # against the one-GPU engine: same logits within the tolerance while the two runs share their history
            s_ids, s_logits = res[0][key + ("one_gpu",)]
            alive = np.ones(d_ids.shape[0], dtype=bool)
            for i in range(N_NEW):
                for b in range(d_ids.shape[0]):
                    if alive[b]:
                        assert rel_err(d_logits[i][0][b], s_logits[i][0][b]) <= tol, (cfg.name, int(strat), i, b)
                alive &= d_ids[:, i] == s_ids[:, i]
            print("%s strategy %d: ties vs oracle %s" % (cfg.name, int(strat), ties))
        np.testing.assert_array_equal(res[0][(cfg.name, "fill")], res[0][(cfg.name, 0)][0])  # device-generated shards = host-loaded shards


# ---------------------------------------------------------------- one sequence: the owner-partitioned kernel across ranks
def _single_configs():
    from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, GPTConfig, MultiHeadAttentionTypeEnums as M, NormEnums as Nm,
                                       PositionEmbeddingEnums as P)
    # L = 2 and L = 4: the launch-to-launch rotation of the residual buffers takes every value; head sizes 32 and 64: both
    # attention forms of the kernel
    return [GPTConfig(name="gqa_l2", L=2, d=256, H=8, Hkv=4, hd=32, F=512, V=1999, norm=Nm.RMSNorm, act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16"),
            GPTConfig(name="gqa_l4", L=4, d=512, H=8, Hkv=2, hd=64, F=1024, V=2003, norm=Nm.LayerNorm, act=A.ReLU, pe=P.RoPE, attn=M.GQA, dtype="float16")]


N_SINGLE = 24


def _single_worker(rank, world, port, q):
    import torch.distributed as dist
    from seq2seqsharp_b200.gpt import DecodingOptions, DecodingStrategyEnums as DS, GPT, synthetic_weights
    from seq2seqsharp_b200.synthetic import prompt_ids
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out = {}
        for cfg in _single_configs():
            w = synthetic_weights(cfg, 5, std=0.05, bias_std=0.02)
            prompt = prompt_ids(9, 1, S_PROMPT, cfg.V)
            opts = DecodingOptions(MaxTgtSentLength=S_PROMPT + N_SINGLE, DecodingStrategy=DS.GreedySearch, BlockedTokens=[0])
            for kernel in ("owner", "streamk"):
                os.environ["TSB200_OWNER"] = "1" if kernel == "owner" else "0"
                gpt = GPT(cfg, device_id=rank, max_batch=1, max_tokens=S_PROMPT + N_SINGLE + 4, tp_rank=rank, tp_size=world)
                gpt.LoadWeights(w)
                gpt.InitComm()
                gpt.Reset()
                ids = np.zeros((1, N_SINGLE), dtype=np.int32)
                logits = []
                ids[:, 0] = gpt.Prefill(prompt, opts)
                logits.append(gpt.Logits())
                for i in range(1, N_SINGLE):
                    ids[:, i] = gpt.Decode(1, opts)[:, 0]
                    logits.append(gpt.Logits())
                path = gpt.DecodePath()
                # a second request on the same engine (the launch counter keeps running) through the graph-replayed loop
                loop = gpt.RunForwardOnSingleDevice(prompt, opts, stop_on_eos=False)
                out[(cfg.name, kernel)] = (ids, logits, path, loop)
                gpt.close()
            os.environ.pop("TSB200_OWNER", None)
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(900)
def test_tensor_parallel_single_sequence_owner_kernel(native, oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from seq2seqsharp_b200.gpt import DecodingOptions, DecodingStrategyEnums as DS, synthetic_weights
    from seq2seqsharp_b200.synthetic import prompt_ids
    from tests.test_gpt_gpu import compare_run, rel_err, tol_for
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_single_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=800) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for cfg in _single_configs():
        w = synthetic_weights(cfg, 5, std=0.05, bias_std=0.02)
        prompt = prompt_ids(9, 1, S_PROMPT, cfg.V)
        opts = DecodingOptions(MaxTgtSentLength=S_PROMPT + N_SINGLE, DecodingStrategy=DS.GreedySearch, BlockedTokens=[0])
        orc = oracle.OracleGPT(cfg, w)
        steps = {}
        o_ids = orc.generate(prompt, opts, uniforms=lambda st, b: oracle.philox_uniform(opts.Seed, opts.SeqBase + b, st),
                             stop_on_eos=False, record=lambda st, lg, p, n: steps.update({st: (lg.copy(), p.copy(), n.copy())}))
        for kernel, want_path in (("owner", 2), ("streamk", 1)):
            ids, logits, path, loop = res[0][(cfg.name, kernel)]
            assert path == want_path, (cfg.name, kernel, path)
            ids1, logits1, path1, loop1 = res[1][(cfg.name, kernel)]
            assert path1 == want_path
            # integer sums (owner) / fixed-order sums (stream-K): every rank holds the same bits
            np.testing.assert_array_equal(ids, ids1)
            for (la, _), (lb, _) in zip(logits, logits1):
                np.testing.assert_array_equal(la, lb)
            np.testing.assert_array_equal(loop, ids)
            np.testing.assert_array_equal(loop1, ids)
            ties = compare_run(oracle, cfg, o_ids, steps, ids, logits, opts, prompt)
            print("%s %s: ties vs oracle %s" % (cfg.name, kernel, ties))
        # the two kernels agree within the tolerance while they share their history
        a_ids, a_logits = res[0][(cfg.name, "owner")][:2]
        b_ids, b_logits = res[0][(cfg.name, "streamk")][:2]
        for i in range(N_SINGLE):
            assert rel_err(a_logits[i][0][0], b_logits[i][0][0]) <= tol_for(cfg), (cfg.name, i)
            if a_ids[0, i] != b_ids[0, i]:
                break
