"""Runs ONE kernel of libtsb200 on a small, L2-exceeding case — the command line that profiler captures use.

    python -m seq2seqsharp_b200.kernel_cases gemv   [--M 1] [--K 4096] [--N 22016] [--dtype f16] [--iters 3]
    python -m seq2seqsharp_b200.kernel_cases decode [--workload c3_b1] [--steps 2]      (whole decode steps, small model)
    python -m seq2seqsharp_b200.kernel_cases topp   [--rows 8] [--V 32000]
    python -m seq2seqsharp_b200.kernel_cases attention [--B 4] [--H 32] [--Hkv 8] [--hd 64] [--T 16384]

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
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def case_gemv(a):
    dt = torch.float16 if a.dtype == "f16" else torch.float32
    nd = N.F16 if a.dtype == "f16" else N.F32
    # several weight matrices are cycled so that consecutive launches never find their weights in L2
    n_mats = max(2, int(300e6 // (a.K * a.N * (2 if a.dtype == "f16" else 4))) + 1)
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


def case_topp(a):
    from .ops import Ops
    g = torch.Generator(device="cuda").manual_seed(0)
    p = torch.softmax(torch.randn(a.rows, a.V, device="cuda", generator=g) * a.spread, dim=-1)
    u = torch.rand(a.rows, generator=torch.Generator().manual_seed(1))
    ms = _time(lambda: Ops.TopPSample(p, a.topP, 0.0, None, u), a.iters)
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
    ap.add_argument("case", choices=["gemv", "decode", "topp", "attention"])
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
    ap.add_argument("--B", type=int, default=4)
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--Hkv", type=int, default=8)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--T", type=int, default=16384)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("kernel_cases needs a GPU (no CPU fallback)")
    torch.cuda.set_device(0)
    {"gemv": case_gemv, "decode": case_decode, "topp": case_topp, "attention": case_attention}[a.case](a)


if __name__ == "__main__":
    main()
