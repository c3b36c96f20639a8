"""Benchmark of the GPT decode hot path on B200 (and of the CPU oracle as the reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

One "step" = one decode step (one new token for each of the B resident sequences) of the workload's model with
its KV cache resident in HBM.  Prints ONE JSON line on rank 0.  For N > 1 launch with torch.distributed.run; each
rank drives its own GPU with its own replica and its own sequences (batch sharding, no collective on the data
path), timing is the max over ranks.

Workloads (synthetic seeded weights and prompts of the named shapes; no dataset is involved):
    c5_b1   Llama-7B-class fp16, B=1,  prompt 512, Top-P 0.95     (headline: latency-bound decode)
    c5_b64  same model, B=64
    c5_b2 .. c5_b8  same model, B=2, 3, 4, 8 (still one persistent launch per step on the fp16 tensor-core variant)
    c3_b1 / c3_b32  Llama-1B-class fp16, prompt 1024, greedy
    c1      tiny fp32 model, B=1, prompt 32, greedy
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    #            config name               B   prompt  strategy  topP
    "c5_b1": ("c5_llama7b_fp16", 1, 512, "topp", 0.95),
    "c5_b64": ("c5_llama7b_fp16", 64, 512, "topp", 0.95),
    "c5_b2": ("c5_llama7b_fp16", 2, 512, "topp", 0.95),
    "c5_b3": ("c5_llama7b_fp16", 3, 512, "topp", 0.95),
    "c5_b4": ("c5_llama7b_fp16", 4, 512, "topp", 0.95),
    "c5_b8": ("c5_llama7b_fp16", 8, 512, "topp", 0.95),
    "c3_b1": ("c3_llama1b_fp16", 1, 1024, "greedy", 1.0),
    "c3_b32": ("c3_llama1b_fp16", 32, 1024, "greedy", 1.0),
    "c2_b8": ("c2_gpt2small_fp16", 8, 128, "topp", 0.9),
    "c1": ("c1_tiny_fp32", 1, 32, "greedy", 1.0),
}
FALLBACK_HBM_GBS = 6650.0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                       "-lms", "200"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        time.sleep(0.25)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def linear_bytes_per_step(cfg, shards=1):
    """Algorithmic bytes of every linear layer of one decode step on ONE GPU: each weight and bias read once; under
    tensor parallelism the layer matrices are cut `shards` ways and the LM head is replicated."""
    es = 2 if cfg.dtype == "float16" else 4
    d, F, V, Hd, KVd = cfg.d, cfg.F, cfg.V, cfg.H * cfg.hd, cfg.kv_heads() * cfg.hd
    nq = Hd + 2 * KVd
    f1 = (2 if cfg.is_glu() else 1) * F
    per_layer = d * nq + nq + Hd * d + d + d * f1 + f1 + F * d + d
    return es * (cfg.L * per_layer // shards + d * V + V)


class CpuSample:
    """Bounded sample of the decode workload on the CPU oracle (the restatement of the reference's TensorSharp.Cpu
    path): models with 1 and 2 of the L layers plus embedding and LM head; per-layer and per-head times are separated
    by the difference and extrapolated linearly to L layers."""

    def __init__(self, cfg, threads):
        import dataclasses

        from oracle import cpu_oracle as O
        self.O, self.cfg = O, cfg
        rng = np.random.default_rng(0)
        self.models = []
        for nl in (1, 2):
            c = dataclasses.replace(cfg, L=nl)
            w = {}
            for name, shape in c.weight_shapes(64).items():
                if name.endswith("m_alpha"):
                    w[name] = np.ones(shape, np.float32)
                elif name.endswith(("m_beta", "m_Bd", "QKVb", ".Qb", ".Kb", ".Vb", ".b0")):
                    w[name] = np.zeros(shape, np.float32)
                else:
                    w[name] = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
            orc = O.OracleGPT(c, w, max_pos=64, threads=threads, faithful_cache=True)
            del w
            ids = rng.integers(1, c.V, size=(1, 8)).astype(np.int32)
            _, p = orc.step(ids)
            self.models.append([orc, O.argmax(p).reshape(1, 1)])

    def measure(self, tokens):
        ts = []
        for m in self.models:
            orc, nxt = m
            if orc.cache_len() > 48:
                orc.reset()
                orc.step(np.ones((1, 8), dtype=np.int32))
            t0 = time.perf_counter()
            for _ in range(tokens):
                _, p = orc.step(nxt)
                nxt = self.O.argmax(p).reshape(1, 1)
            ts.append((time.perf_counter() - t0) / tokens)
            m[1] = nxt
        per_layer = max(ts[1] - ts[0], 1e-9)
        head = max(ts[0] - per_layer, 0.0)
        return 1.0 / (head + self.cfg.L * per_layer)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_oracle as O
    from seq2seqsharp_b200.configs import CONFIGS
    name, B, S, strat, topP = WORKLOADS[args.workload]
    cfg = CONFIGS[name]
    threads = O.max_threads()
    sample_run = CpuSample(cfg, threads)
    vals = []
    t_start = time.perf_counter()
    tps = 0.0
    for i in range(args.warmup + args.steps):
        tps = sample_run.measure(2)
        if i >= args.warmup:
            vals.append(tps)
        if time.perf_counter() - t_start > 200:
            break
    v = float(statistics.median(vals)) if vals else float(tps)
    sample = ("CPU oracle (C++ restatement of the reference's TensorSharp.Cpu fp32 path; the C# reference cannot run here), B=1: "
              "1- and 2-layer models + embedding + LM head, 2 decode steps each per bench step, extrapolated linearly to %d layers" % cfg.L)
    line = {"impl": "reference", "metric": "decode tokens/s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": args.warmup, "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "model": name, "batch_per_gpu": 1, "prompt_len": S},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


def run_b200(args):
    import torch
    import torch.distributed as dist

    from seq2seqsharp_b200 import _native
    from seq2seqsharp_b200.configs import CONFIGS, SEED
    from seq2seqsharp_b200.gpt import DecodingOptions, DecodingStrategyEnums, GPT
    from seq2seqsharp_b200.synthetic import prompt_ids

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    if not _native.lib().TSB200_IsAvailable(local):
        raise RuntimeError("bench: device %d is not an sm_100 GPU; this backend has no CPU fallback" % local)

    name, B, S, strat, topP = WORKLOADS[args.workload]
    cfg = CONFIGS[name]
    K, W = args.steps, max(args.warmup, 3)
    n_prof = 8
    max_tokens = S + W + 2 * K + n_prof + 16
    tp = args.parallelism == "tp" and world > 1
    gpt = GPT(cfg, device_id=local, max_batch=B, max_tokens=max_tokens, tp_rank=rank if tp else 0, tp_size=world if tp else 1)
    gpt.FillSynthetic(SEED, 0.02, 0.0)
    if tp:
        gpt.InitComm()
    prompt = prompt_ids(SEED + (0 if tp else rank), B, S, cfg.V)
    opts = DecodingOptions(MaxTgtSentLength=max_tokens, BlockedTokens=[0], TopP=topP, Temperature=1.0, RepeatPenalty=2.0,
                           DecodingStrategy=DecodingStrategyEnums.Sampling if strat == "topp" else DecodingStrategyEnums.GreedySearch,
                           Seed=SEED, SeqBase=0 if tp else rank * B)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    lib = _native.lib()

    def launches():
        import ctypes as C
        n = C.c_int64(0)
        lib.TSB200_LaunchCount(local, C.byref(n))
        return n.value

    # prefill (device-timed; reported beside the decode metric)
    gpt.Reset()
    first = gpt.Prefill(prompt, opts)
    prefill_ms, _ = gpt.LastTiming()
    prefill_ms = max_over_ranks(prefill_ms)
    gpt.Decode(W, opts)  # warm-up (also captures the step graph)

    # ---- timed region: K graph-replayed decode steps, ids fed back on the device, inputs resident in HBM
    gpt.EnableStepTiming(True)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    l0 = launches()
    t_wall0 = time.perf_counter()
    ids = gpt.Decode(K, opts)
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall0
    ms, _ = gpt.LastTiming()
    n_launch = launches() - l0
    barrier()
    ms = max_over_ranks(ms)
    step_ms = gpt.StepTimes(K)
    gpt.EnableStepTiming(False)
    T_mid = S + W + K // 2

    # ---- end to end through the public API with HOST buffers: ids H2D, step, ids D2H, every step
    last = ids[:, -1].copy()
    gpt.StepHost(last, opts)  # warm
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        last = gpt.StepHost(last, opts)
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    e2e_s = max_over_ranks(e2e_s)

    # ---- roofline of the dominant kernel class (the decode GEMV): CUDA events around every launch, un-captured
    T_prof = gpt.CacheLength() + n_prof // 2
    prof = gpt.ProfileDecode(n_prof, opts)
    lin_ms, lin_groups = prof["linear"]
    lin_bytes = linear_bytes_per_step(cfg, world if tp else 1)
    dominant = "gemv_stream_kernel / gemm_tc_kernel (all linear layers of a decode step)"
    if prof["decode_stack"][1] > 0:
        # batch <= 4: one persistent launch per step runs every linear plus RoPE, cache append and attention; its
        # algorithmic bytes are the weights once plus the KV cache read and the appended rows
        lin_ms, lin_groups = prof["decode_stack"]
        es = 2 if cfg.dtype == "float16" else 4
        lin_bytes += B * cfg.L * 2 * (cfg.kv_heads() // (world if tp else 1)) * cfg.hd * (T_prof + 1) * es
        dominant = "decode_stack_kernel (persistent: all linears, RoPE, cache append and attention of a decode step)"
    hbm, which = peaks()
    achieved = (lin_bytes * n_prof / 1e9) / (lin_ms / 1e3) if lin_ms > 0 else 0.0
    traffic = None
    traffic_path = os.path.join(ROOT, "profiles", "gemv_traffic.json")
    if os.path.exists(traffic_path):
        with open(traffic_path) as fh:
            tj = json.load(fh)
        # dram bytes per algorithmic byte measured by ncu on the same kernel, scaled to one launch of this workload
        ratio = tj.get("dram_bytes_per_algorithmic_byte", 0)
        if prof["decode_stack"][1] == 0:
            ratio = tj.get("per_linear_kernel", {}).get("dram_bytes_per_algorithmic_byte", ratio)
        traffic = ratio * lin_bytes / max(1, lin_groups // n_prof) or None
    step_bytes = gpt.StepBytes(B, T_mid)
    seqs = B if tp else world * B      # sequences decoded by the whole job
    tokens = seqs * K
    value = tokens / (ms / 1e3)
    line = {
        "metric": "decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
        "dtype": "f16" if cfg.dtype == "float16" else "f32", "data": "synthetic",
        "config": {"workload": args.workload, "model": name, "batch_per_gpu": B, "prompt_len": S, "context_at_timing": T_mid,
                   "decoding": strat, "topP": topP,
                   "parallelism": ("tensor-parallel x%d (heads and FFN sharded, 2 all-reduces per layer)" % world) if tp else "batch-sharded replicas x%d" % world,
                   "l2": "inputs larger than L2: %.0f MB of weights+KV streamed per step vs 126 MB L2" % (step_bytes / 1e6)},
        "e2e": {"value": seqs * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": B * 4 + 12, "d2h_bytes_per_step": B * 4},
        "gpu_launches": int(n_launch),
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved,
                     "peak": hbm, "peak_source": which, "unit": "GB/s", "frac": achieved / hbm,
                     "traffic": traffic, "algorithmic_bytes_per_launch": lin_bytes / max(1, lin_groups // n_prof),
                     "launches_per_step": lin_groups // n_prof},
        "step_roofline": {"algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes * K / 1e9 / (ms / 1e3),
                          "frac_of_hbm_peak": step_bytes * K / 1e9 / (ms / 1e3) / hbm},
        "p50_ms_per_token": float(np.median(step_ms)) if len(step_ms) else None,
        "prefill": {"tokens_per_s": seqs * S / (prefill_ms / 1e3), "ms": prefill_ms},
        "kernel_classes_ms_per_step": {k: v[0] / n_prof for k, v in prof.items()},
        "host_wall_ms_per_step": 1e3 * t_wall / K,
    }
    if world == 1 and not tp and S >= 16:
        # outside the timed region: a request whose prompt head is parked (restore + run the rest) against the full prefill
        head = S - 32 if S > 64 else S // 2
        gpt.Reset()
        gpt.Prefill(prompt[:, :head], opts)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        snap = gpt.CacheSnapshot()
        torch.cuda.synchronize()
        snap_ms = 1e3 * (time.perf_counter() - t0)
        gpt.Reset()
        t0 = time.perf_counter()
        gpt.CacheRestore(snap)
        torch.cuda.synchronize()
        restore_ms = 1e3 * (time.perf_counter() - t0)
        gpt.Extend(prompt[:, head:], opts)
        ext_ms, _ = gpt.LastTiming()
        line["cache_reuse"] = {"cached_tokens": head, "suffix_tokens": S - head, "snapshot_bytes": snap.nbytes,
                               "snapshot_ms_wall": snap_ms, "restore_ms_wall": restore_ms, "suffix_ms": ext_ms,
                               "full_prefill_ms": prefill_ms}
        snap.close()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import cpu_oracle as O
        thr = O.max_threads()
        v_all = CpuSample(cfg, thr).measure(4)
        v_one = CpuSample(cfg, 1).measure(2)
        line["cpu_baseline"] = {
            "value": v_all, "unit": "tokens/s", "cores": thr, "kind": "port", "value_1_thread": v_one,
            "sample": "CPU oracle (restatement of the reference's TensorSharp.Cpu fp32 path, reference-style realloc+copy KV cache), B=1: "
                      "1- and 2-layer models + embedding + LM head timed over 4 decode steps each, extrapolated linearly to %d layers; "
                      "1-thread figure matches the reference's single-threaded managed SGEMM" % cfg.L}
    if rank == 0:
        print(json.dumps(line))
    gpt.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5_b1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallelism", default="replicas", choices=["replicas", "tp"],
                    help="N > 1: 'replicas' = batch-sharded independent sequences (weak scaling, the default); "
                         "'tp' = one model sharded over the GPUs with two all-reduces per layer (strong scaling)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
