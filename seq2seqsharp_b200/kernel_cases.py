"""Runs ONE kernel of libtsb200 on a small, L2-exceeding case — the command line that profiler captures use.

    python -m seq2seqsharp_b200.kernel_cases gemv   [--M 1] [--K 4096] [--N 22016] [--dtype f16] [--iters 3]
    python -m seq2seqsharp_b200.kernel_cases decode [--workload c3_b1] [--steps 2]      (whole decode steps, small model)
    python -m seq2seqsharp_b200.kernel_cases topp   [--rows 8] [--V 32000]
    python -m seq2seqsharp_b200.kernel_cases attention [--B 4] [--H 32] [--Hkv 8] [--hd 64] [--T 16384]
    python -m seq2seqsharp_b200.kernel_cases beam   [--workload c3_b1] [--B 1] [--beams 4] [--prompt 1024] [--steps 32]

Each case prints its own CUDA-event timing and the algorithmic bytes it moves, so a capture and a plain run can be
compared.  Device buffers are torch tensors; every kernel is reached through the C ABI.
"""
import argparse
import ctypes as C
import sys

import numpy as np
import torch

from . import _native as N


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _time(fn, iters):
    """Average device time of one call: `iters` calls are captured into one CUDA graph (so host launch overhead is
    not on the clock) and the graph is timed with CUDA events on the launching stream."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def case_gemv(a):
    dt = torch.float16 if a.dtype == "f16" else torch.float32
    nd = N.F16 if a.dtype == "f16" else N.F32
    # several weight matrices are cycled so that consecutive launches never find their weights in L2
    n_mats = max(3, int(1.2e9 // (a.K * a.N * (2 if a.dtype == "f16" else 4))) + 1)
    Ws = [(torch.randn(a.K, a.N, device="cuda") * 0.02).to(dt) for _ in range(n_mats)]
    x = torch.randn(a.M, a.K, device="cuda").to(dt)
    b = torch.zeros(a.N, device="cuda", dtype=dt)
    y = torch.empty(a.M, a.N, device="cuda", dtype=dt)
    wsb = N.lib().TSB200_LinearWorkspaceBytes(a.M, a.K, a.N)
    ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
    i = [0]

    def run():
        W = Ws[i[0] % n_mats]
        i[0] += 1
        N.call("TSB200_LinearBiasAct", 0, nd, y.data_ptr(), None, x.data_ptr(), W.data_ptr(), b.data_ptr(), None, a.M, a.K, a.N,
               N.ACT_NONE, ws.data_ptr(), wsb, _stream())

    ms = _time(run, a.iters)
    nbytes = a.K * a.N * W_es(a) + a.N * W_es(a)
    print("gemv M=%d K=%d N=%d %s: %.3f ms/launch, %.1f GB/s algorithmic (%d matrices cycled)" % (a.M, a.K, a.N, a.dtype, ms, nbytes / ms / 1e6, n_mats))


def case_gemv_packed(a):
    """The engine's TMA-fed streaming GEMV on packed tiles (M <= 4), optionally with the fused RMSNorm prologue."""
    dt = torch.float16 if a.dtype == "f16" else torch.float32
    nd = N.F16 if a.dtype == "f16" else N.F32
    es = W_es(a)
    pb = N.lib().TSB200_PackedWeightBytes(nd, a.K, a.N)
    n_mats = max(3, int(1.2e9 // pb) + 1)
    W = (torch.randn(a.K, a.N, device="cuda") * 0.02).to(dt)
    Wps = []
    for _ in range(n_mats):
        Wp = torch.empty(pb, dtype=torch.uint8, device="cuda")
        N.call("TSB200_PackWeight", 0, nd, Wp.data_ptr(), W.data_ptr(), nd, a.K, a.N, _stream())
        Wps.append(Wp)
    x = torch.randn(a.M, a.K, device="cuda").to(dt)
    x32 = torch.randn(a.M, a.K, device="cuda")
    gamma = torch.ones(a.K, device="cuda", dtype=dt)
    b = torch.zeros(a.N, device="cuda", dtype=dt)
    y = torch.empty(a.M, a.N, device="cuda", dtype=dt)
    wsb = N.lib().TSB200_LinearPackedWorkspaceBytes(nd, a.M, a.K, a.N)
    ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
    i = [0]

    def run():
        Wp = Wps[i[0] % n_mats]
        i[0] += 1
        N.call("TSB200_LinearPacked", 0, nd, y.data_ptr(), None, None if a.norm else x.data_ptr(), x32.data_ptr() if a.norm else None,
               gamma.data_ptr() if a.norm else None, None, 1 if a.norm else -1, 1e-6, Wp.data_ptr(), b.data_ptr(), None, a.M, a.K, a.N,
               N.ACT_NONE, ws.data_ptr(), wsb, _stream())

    ms = _time(run, a.iters)
    nbytes = a.K * a.N * es + a.N * es
    print("gemv_packed M=%d K=%d N=%d %s norm=%d: %.4f ms/launch, %.1f GB/s algorithmic (%d matrices cycled)" % (
        a.M, a.K, a.N, a.dtype, a.norm, ms, nbytes / ms / 1e6, n_mats))


def W_es(a):
    return 2 if a.dtype == "f16" else 4


def case_decode(a):
    from .configs import CONFIGS, SEED
    from .gpt import DecodingOptions, DecodingStrategyEnums, GPT
    from .synthetic import prompt_ids
    sys.path.insert(0, ".")
    from bench import WORKLOADS
    name, B, S, strat, topP = WORKLOADS[a.workload]
    cfg = CONFIGS[name]
    S = min(S, a.prompt)
    gpt = GPT(cfg, max_batch=B, max_tokens=S + a.steps + 16)
    gpt.FillSynthetic(SEED, 0.02, 0.0)
    opts = DecodingOptions(MaxTgtSentLength=S + a.steps + 8, BlockedTokens=[0], TopP=topP,
                           DecodingStrategy=DecodingStrategyEnums.Sampling if strat == "topp" else DecodingStrategyEnums.GreedySearch)
    gpt.Prefill(prompt_ids(SEED, B, S, cfg.V), opts)
    gpt.Decode(a.steps, opts)
    ms, n = gpt.LastTiming()
    print("decode %s: %d steps, %.3f ms/step, %d launches" % (a.workload, a.steps, ms / a.steps, n))
    gpt.close()


def case_beam(a):
    """Beam search on a benchmark configuration: wall time per step (a forward of one token per hypothesis, the candidate
    kernel, the host's selection and the cache copies of that step)."""
    import time
    from .beam import beam_search
    from .configs import CONFIGS, SEED
    from .gpt import DecodingOptions, DecodingStrategyEnums, GPT
    from .synthetic import prompt_ids
    sys.path.insert(0, ".")
    from bench import WORKLOADS
    name, _, S, _, _ = WORKLOADS[a.workload]
    cfg = CONFIGS[name]
    S = min(S, a.prompt)
    B, K = a.B, a.beams
    gpt = GPT(cfg, max_batch=B * K, max_tokens=S + a.steps + 16)
    gpt.FillSynthetic(SEED, 0.02, 0.0)
    opts = DecodingOptions(MaxTgtSentLength=S + a.steps, BlockedTokens=[0], BeamSearchSize=K,
                           DecodingStrategy=DecodingStrategyEnums.GreedySearch)
    prompts = prompt_ids(SEED, B, S, cfg.V)
    beam_search(gpt, prompts, DecodingOptions(MaxTgtSentLength=S + 3, BlockedTokens=[0], BeamSearchSize=K))   # warm-up: graphs, scratch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = beam_search(gpt, prompts, opts)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    print("beam search %s: %d prompts of %d tokens x %d beams, %d steps in %.1f ms (prefill included): %.3f ms/step wall, %d sequence copies" % (
        a.workload, B, S, K, res.steps, dt * 1e3, dt * 1e3 / max(1, res.steps), res.copies))
    gpt.close()


def case_topp(a):
    from .ops import Ops
    g = torch.Generator(device="cuda").manual_seed(0)
    p = torch.softmax(torch.randn(a.rows, a.V, device="cuda", generator=g) * a.spread, dim=-1)
    u = torch.rand(a.rows, generator=torch.Generator().manual_seed(1))
    out = torch.empty(a.rows, dtype=torch.int32, device="cuda")
    wsb = N.lib().TSB200_TopPWorkspaceBytes(a.rows, a.V)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    ud = u.cuda()
    hist = torch.arange(1, a.hist + 1, dtype=torch.int32, device="cuda").repeat(a.rows, 1).contiguous() if a.hist else None
    hlen = torch.full((a.rows,), a.hist, dtype=torch.int32, device="cuda") if a.hist else None
    ms = _time(lambda: N.call("TSB200_TopPSample", 0, out.data_ptr(), p.data_ptr(), a.rows, a.V, a.topP, 2.0 if a.hist else 0.0,
                              hist.data_ptr() if a.hist else None, hlen.data_ptr() if a.hist else None, a.hist, ud.data_ptr(),
                              ws.data_ptr(), wsb, _stream()), a.iters)
    print("topp rows=%d V=%d topP=%g: %.3f ms/launch" % (a.rows, a.V, a.topP, ms))


def case_attention(a):
    dt = torch.float16 if a.dtype == "f16" else torch.float32
    nd = N.F16 if a.dtype == "f16" else N.F32
    Tmax = a.T + 8
    cK = torch.randn(a.B, a.Hkv, Tmax, a.hd, device="cuda").to(dt)
    cV = torch.randn(a.B, a.Hkv, Tmax, a.hd, device="cuda").to(dt)
    q = torch.randn(a.B, a.H * a.hd, device="cuda").to(dt)
    out = torch.empty(a.B, a.H, a.hd, device="cuda", dtype=dt)
    wsb = N.lib().TSB200_FlashDecodeWorkspaceBytes(a.B, a.H, a.hd, a.T)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    ms = _time(lambda: N.call("TSB200_FlashDecode", 0, nd, out.data_ptr(), q.data_ptr(), a.H * a.hd, cK.data_ptr(), cV.data_ptr(), a.B,
                              a.H, a.Hkv, a.hd, a.T, Tmax, ws.data_ptr(), wsb, _stream()), a.iters)
    nbytes = 2 * a.B * a.Hkv * a.T * a.hd * W_es(a)
    print("flash-decode B=%d H=%d Hkv=%d hd=%d T=%d: %.3f ms/launch, %.1f GB/s algorithmic" % (a.B, a.H, a.Hkv, a.hd, a.T, ms, nbytes / ms / 1e6))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemv", "gemv_packed", "decode", "topp", "attention", "beam"])
    ap.add_argument("--norm", type=int, default=0)
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=22016)
    ap.add_argument("--dtype", default="f16")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--workload", default="c3_b1")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--V", type=int, default=32000)
    ap.add_argument("--topP", type=float, default=0.95)
    ap.add_argument("--spread", type=float, default=0.05)
    ap.add_argument("--hist", type=int, default=0)
    ap.add_argument("--B", type=int, default=4)
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--Hkv", type=int, default=8)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--T", type=int, default=16384)
    ap.add_argument("--beams", type=int, default=4)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("kernel_cases needs a GPU (no CPU fallback)")
    torch.cuda.set_device(0)
    {"gemv": case_gemv, "gemv_packed": case_gemv_packed, "decode": case_decode, "topp": case_topp, "attention": case_attention, "beam": case_beam}[a.case](a)


if __name__ == "__main__":
    main()
