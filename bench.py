"""Benchmark of the GPT decode hot path on B200 (and of the CPU oracle as the reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

One "step" = one decode step (one new token for each of the B resident sequences) of the workload's model with
its KV cache resident in HBM.  Prints ONE JSON line on rank 0.  For N > 1 launch with torch.distributed.run; each
rank drives its own GPU with its own replica and its own sequences (batch sharding, no collective on the data
path), timing is the max over ranks.

Workloads (synthetic seeded weights and prompts of the named shapes; no dataset is involved):
    c5_b1   Llama-7B-class fp16, B=1,  prompt 512, Top-P 0.95     (headline: latency-bound decode)
    c5_b64  same model, B=64
    c5_b2 .. c5_b8  same model, B=2, 3, 4, 8 (one launch per operation on the tensor-core streaming linears)
    c3_b1 / c3_b2 / c3_b4 / c3_b8 / c3_b32  Llama-1B-class fp16, prompt 1024, greedy
    c4_b4   the same 1B-class model, B=4, 16384-token prompts, greedy (long-context KV-cache stress)
    c1      tiny fp32 model, B=1, prompt 32, greedy

With N > 1 the 7B-class workloads (c5_*) run ONE model tensor-parallel over the N GPUs (strong scaling: `value` is the
tokens/s of the one sharded model); the other workloads run N batch-sharded replicas (weak scaling).  `--parallelism`
overrides.  After the timed region the benchmarked engine is checked against an independent engine (one GPU, one launch
per operation) fed the same ids (`parity_check`; the run fails above the dtype's logit tolerance), and on one GPU a
`secondary` block reports the large-batch decode and prefill figures the metric also names, a small batch, the long-context
configuration and a batch of sequences of different lengths.
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
    "c3_b2": ("c3_llama1b_fp16", 2, 1024, "greedy", 1.0),
    "c3_b4": ("c3_llama1b_fp16", 4, 1024, "greedy", 1.0),
    "c3_b8": ("c3_llama1b_fp16", 8, 1024, "greedy", 1.0),
    "c3_b32": ("c3_llama1b_fp16", 32, 1024, "greedy", 1.0),
    "c4_b4": ("c4_llama1b_longctx_fp16", 4, 16384, "greedy", 1.0),
    "c2_b8": ("c2_gpt2small_fp16", 8, 128, "topp", 0.9),
    "c1": ("c1_tiny_fp32", 1, 32, "greedy", 1.0),
}
FALLBACK_HBM_GBS = 6650.0


FALLBACK_TFLOPS = 1590.0          # burst; sustained under the power cap settles near 1400
FALLBACK_TFLOPS_SUSTAINED = 1400.0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def tensor_peaks():
    """(burst, sustained) dense bf16/fp16 TFLOP/s and where they come from."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as fh:
            d = json.load(fh)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return FALLBACK_TFLOPS, FALLBACK_TFLOPS_SUSTAINED, "fallback"


def prefill_flops(cfg, B, S):
    """Algorithmic flops of a prefill: every layer's matmuls on B*S rows, the LM head on the last row of each sequence,
    causal attention (QK^T and PV over S^2 / 2 pairs)."""
    d, F, V, Hd, KVd = cfg.d, cfg.F, cfg.V, cfg.H * cfg.hd, cfg.kv_heads() * cfg.hd
    per_layer = d * (Hd + 2 * KVd) + Hd * d + (3 if cfg.is_glu() else 2) * d * F
    return 2.0 * B * S * cfg.L * per_layer + 2.0 * B * d * V + 4.0 * B * cfg.L * cfg.H * cfg.hd * S * S / 2.0


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
    path).  Small models (under 2e8 matmul parameters: the tiny fp32 and the GPT-2-small-shaped configurations) are
    timed in full.  For the larger ones models with 1 and 2 of the L layers plus embedding and LM head are timed;
    per-layer and per-head times are separated by the difference and extrapolated linearly to L layers."""

    def __init__(self, cfg, threads):
        import dataclasses

        from oracle import cpu_oracle as O
        self.O, self.cfg = O, cfg
        self.full = cfg.matmul_params() < 2e8
        rng = np.random.default_rng(0)
        self.models = []
        for nl in ((cfg.L,) if self.full else (1, 2)):
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

    def describe(self):
        if self.full:
            return "the full %d-layer model, 8-token context" % self.cfg.L
        return ("1- and 2-layer models + embedding + LM head, 8-token context, extrapolated linearly to %d layers" % self.cfg.L)

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
        if self.full:
            return 1.0 / ts[0]
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
              "%s, 2 decode steps per bench step" % sample_run.describe())
    line = {"impl": "reference", "metric": "decode tokens/s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": args.warmup, "ms_per_step": 1000.0 / v, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "model": name, "batch_per_gpu": 1, "prompt_len": S},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


def make_options(strat, topP, max_tokens, seed, seq_base):
    from seq2seqsharp_b200.gpt import DecodingOptions, DecodingStrategyEnums
    return DecodingOptions(MaxTgtSentLength=max_tokens, BlockedTokens=[0], TopP=topP, Temperature=1.0, RepeatPenalty=2.0,
                           DecodingStrategy=DecodingStrategyEnums.Sampling if strat == "topp" else DecodingStrategyEnums.GreedySearch,
                           Seed=seed, SeqBase=seq_base)


def per_operation_engine(cfg, device, max_batch, max_tokens, seed):
    """An independent engine on ONE GPU that decodes with one launch per operation and none of the fusions of the
    benchmarked path (no persistent decode-step kernel, no tensor parallelism; separate norm and RoPE-append launches; up to
    four rows on the FMA streaming GEMV instead of the tensor-core kernel): the checker of the benchmarked engine."""
    from seq2seqsharp_b200.gpt import GPT
    knobs = {"TSB200_STACK": "0", "TSB200_FUSED_STEP": "0", "TSB200_GEMV_MAXROWS": "4"}    # read when the engine is created
    old = {k: os.environ.get(k) for k in knobs}
    os.environ.update(knobs)
    try:
        ref = GPT(cfg, device_id=device, max_batch=max_batch, max_tokens=max_tokens)
    finally:
        for k, v in old.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v
    ref.FillSynthetic(seed, 0.02, 0.0)
    return ref


def parity_check(gpt, ref, prompt, opts, n_steps, tol):
    """Both engines prefill the same prompt and then take n_steps decode steps fed the SAME ids (the benchmarked engine's
    own choices, through the host-buffer step).  Compares the logits of every step relative to the step's largest
    |logit|.  `ref` is None on ranks that only take part in a tensor-parallel engine's collective steps."""
    worst, where = 0.0, None

    def cmp(step):
        nonlocal worst, where
        if ref is None:
            return
        la, lb = gpt.Logits(want_probs=False)[0], ref.Logits(want_probs=False)[0]
        e = float(np.abs(la - lb).max() / max(1e-12, float(np.abs(lb).max())))
        if not np.isfinite(la).all():
            e = float("inf")
        if e > worst:
            worst, where = e, step
    gpt.Reset()
    last = gpt.Prefill(prompt, opts)
    if ref is not None:
        ref.Reset()
        ref.Prefill(prompt, opts)
    cmp(0)
    ids_equal = True
    for i in range(n_steps):
        nxt = gpt.StepHost(last, opts)
        if ref is not None:
            r = ref.StepHost(last, opts)
            ids_equal = ids_equal and bool((r == nxt).all())
        cmp(i + 1)
        last = nxt
    return {"max_rel_logit_err": worst, "at_step": where, "steps": n_steps + 1, "tolerance": tol, "ids_equal": ids_equal,
            "ok": bool(worst <= tol), "against": "one-GPU engine with one unfused launch per operation, fed the same ids"}


def measure_secondary(local, name, B, S, strat, topP, steps=16, warm=3, want_prefill=False):
    """One more workload, outside the headline timed region: graph-replayed decode tokens/s with the linear layers' HBM
    and tensor-pipe fractions, and (optionally) the prefill's TFLOP/s."""
    import torch

    from seq2seqsharp_b200.configs import CONFIGS, SEED
    from seq2seqsharp_b200.gpt import GPT
    from seq2seqsharp_b200.synthetic import prompt_ids
    cfg = CONFIGS[name]
    n_prof = 4
    max_tokens = S + warm + steps + n_prof + 8
    gpt = GPT(cfg, device_id=local, max_batch=B, max_tokens=max_tokens)
    gpt.FillSynthetic(SEED, 0.02, 0.0)
    prompt = prompt_ids(SEED, B, S, cfg.V)
    opts = make_options(strat, topP, max_tokens, SEED, 0)
    gpt.Reset()
    gpt.Prefill(prompt, opts)
    if want_prefill:   # second run: the first one paid one-time set-up (kernel attributes, tensor maps)
        gpt.Reset()
        gpt.Prefill(prompt, opts)
    prefill_ms, _ = gpt.LastTiming()
    gpt.Decode(warm, opts)
    gpt.Decode(steps, opts)
    torch.cuda.synchronize()
    ms, _ = gpt.LastTiming()
    T_mid = S + warm + steps // 2
    prof = gpt.ProfileDecode(n_prof, opts)
    hbm, _ = peaks()
    burst, sustained, which = tensor_peaks()
    out = {"workload": "%s B=%d prompt %d %s" % (name, B, S, strat), "decode_tokens_per_s": B * steps / (ms / 1e3),
           "ms_per_step": ms / steps, "context_at_timing": T_mid,
           "step_frac_of_hbm_peak": gpt.StepBytes(B, T_mid) * steps / 1e9 / (ms / 1e3) / hbm,
           "kernel_classes_ms_per_step": {k: v[0] / n_prof for k, v in prof.items() if v[1] > 0}}
    lin_ms = (prof["linear"][0] + prof["decode_stack"][0]) / n_prof
    if lin_ms > 0:
        flops = 2.0 * B * cfg.matmul_params()
        out["linear_layers"] = {"ms_per_step": lin_ms, "hbm_gbs": linear_bytes_per_step(cfg) / 1e9 / (lin_ms / 1e3),
                                "frac_of_hbm_peak": linear_bytes_per_step(cfg) / 1e9 / (lin_ms / 1e3) / hbm,
                                "tflops": flops / 1e12 / (lin_ms / 1e3),
                                "frac_of_tensor_peak_sustained": flops / 1e12 / (lin_ms / 1e3) / sustained}
    if prof["attention"][1] > 0:
        es = 2 if cfg.dtype == "float16" else 4
        kv = B * cfg.L * 2 * cfg.kv_heads() * cfg.hd * (gpt.CacheLength() - n_prof // 2) * es
        a_ms = prof["attention"][0] / n_prof
        out["attention"] = {"ms_per_step": a_ms, "kv_gbs": kv / 1e9 / (a_ms / 1e3), "frac_of_hbm_peak": kv / 1e9 / (a_ms / 1e3) / hbm}
    if want_prefill:
        fl = prefill_flops(cfg, B, S)
        out["prefill"] = {"tokens": B * S, "ms": prefill_ms, "tokens_per_s": B * S / (prefill_ms / 1e3), "tflops": fl / 1e12 / (prefill_ms / 1e3),
                          "frac_of_tensor_peak_sustained": fl / 1e12 / (prefill_ms / 1e3) / sustained,
                          "frac_of_tensor_peak_burst": fl / 1e12 / (prefill_ms / 1e3) / burst, "peak_source": which}
    gpt.close()
    return out


def measure_mixed_batch(local, name, lens, steps=16, warm=3, new_prompt=128):
    """Sequences of different lengths in one batch (outside the headline timed region): prompts of `lens` tokens in one
    padded prefill, graph-replayed decode with a cache length per sequence, and one slot handed to a new request (park
    the old sequence, reset the slot, run the newcomer's prompt) while the others keep their state."""
    import time

    import torch

    from seq2seqsharp_b200.configs import CONFIGS, SEED
    from seq2seqsharp_b200.gpt import GPT
    from seq2seqsharp_b200.synthetic import prompt_ids
    cfg = CONFIGS[name]
    B, S = len(lens), max(lens)
    max_tokens = S + warm + 2 * steps + 16
    gpt = GPT(cfg, device_id=local, max_batch=B, max_tokens=max_tokens)
    gpt.FillSynthetic(SEED, 0.02, 0.0)
    full = prompt_ids(SEED, B, S, cfg.V)
    prompts = [list(map(int, full[b, :n])) for b, n in enumerate(lens)]
    opts = make_options("topp", 0.95, max_tokens, SEED, 0)
    gpt.PrefillRagged(prompts, opts)
    gpt.Reset()
    gpt.PrefillRagged(prompts, opts)      # second run: the first one paid one-time set-up
    prefill_ms, _ = gpt.LastTiming()
    gpt.Decode(warm, opts)
    gpt.Decode(steps, opts)
    torch.cuda.synchronize()
    ms, _ = gpt.LastTiming()
    # the shortest sequence leaves, another request takes its slot
    slot = int(np.argmin(lens))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    snap = gpt.SlotSnapshot(slot)
    torch.cuda.synchronize()
    park_ms = 1e3 * (time.perf_counter() - t0)
    gpt.SlotReset(slot)
    gpt.SlotExtend(slot, prompt_ids(SEED + 1, 1, new_prompt, cfg.V)[0], opts)
    refill_ms, _ = gpt.LastTiming()
    gpt.Decode(steps, opts)
    torch.cuda.synchronize()
    ms2, _ = gpt.LastTiming()
    out = {"workload": "%s, %d sequences with prompts of %s tokens, topp" % (name, B, "/".join(map(str, lens))),
           "prefill_ms": prefill_ms, "prefill_tokens": int(sum(lens)), "padded_tokens": B * S,
           "decode_tokens_per_s": B * steps / (ms / 1e3), "ms_per_step": ms / steps, "decode_path": gpt.DecodePath(),
           "slot_refill": {"park_ms_wall": park_ms, "parked_bytes": snap.nbytes, "new_prompt_tokens": new_prompt, "prompt_ms": refill_ms,
                           "decode_ms_per_step_after": ms2 / steps},
           "cache_lengths_at_end": [int(x) for x in gpt.CacheLengths()]}
    snap.close()
    gpt.close()
    return out


def run_b200(args):
    import torch
    import torch.distributed as dist

    from seq2seqsharp_b200 import _native
    from seq2seqsharp_b200.configs import CONFIGS, SEED
    from seq2seqsharp_b200.gpt import GPT
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
    n_check = 8
    max_tokens = S + W + 2 * K + n_prof + 16
    par = args.parallelism
    if par == "auto":   # the 7B-class model is sharded over the GPUs; smaller models run as batch-sharded replicas
        par = "tp" if (world > 1 and args.workload.startswith("c5_") and cfg.kv_heads() % world == 0) else "replicas"
    tp = par == "tp" and world > 1
    gpt = GPT(cfg, device_id=local, max_batch=B, max_tokens=max_tokens, tp_rank=rank if tp else 0, tp_size=world if tp else 1)
    gpt.FillSynthetic(SEED, 0.02, 0.0)
    if tp:
        gpt.InitComm()
    prompt = prompt_ids(SEED + (0 if tp else rank), B, S, cfg.V)
    opts = make_options(strat, topP, max_tokens, SEED, 0 if tp else rank * B)

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

    # prefill (device-timed; reported beside the decode metric).  The first prefill pays one-time set-up (kernel
    # attributes, tensor maps, and under tensor parallelism NCCL's first collective), so it is run twice.
    gpt.Reset()
    gpt.Prefill(prompt, opts)
    first_prefill_ms, _ = gpt.LastTiming()
    barrier()
    gpt.Reset()
    gpt.Prefill(prompt, opts)
    prefill_ms, _ = gpt.LastTiming()
    prefill_ms = max_over_ranks(prefill_ms)
    gpt.Decode(W, opts)  # warm-up (also captures the step graph)

    # ---- timed region: K graph-replayed decode steps, ids fed back on the device, inputs resident in HBM
    gpt.EnableStepTiming(True)
    sampler = ClockSampler(local)
    sampler.start()   # before the barrier: spawning the sampler takes milliseconds, and under tensor parallelism a rank that
    barrier()         # starts late makes the others wait inside their first step
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
    barrier()
    T_prof = gpt.CacheLength() + n_prof // 2
    prof = gpt.ProfileDecode(n_prof, opts)
    es = 2 if cfg.dtype == "float16" else 4
    lin_ms, lin_groups = prof["linear"]
    lin_bytes = linear_bytes_per_step(cfg, world if tp else 1)
    dominant = ("gemm_stream_mma_kernel / gemm_stream_tc_kernel (all linear layers of a decode step: q|k|v with norm, RoPE and cache "
                "append, out-projection, FFN-up with norm, FFN-down, LM head; timed launch by launch outside the graph)")
    if prof["decode_stack"][1] > 0:
        # one persistent launch per step runs every linear plus RoPE, cache append and attention; its
        # algorithmic bytes are the weights once plus the KV cache read and the appended rows
        lin_ms, lin_groups = prof["decode_stack"]
        lin_bytes += B * cfg.L * 2 * (cfg.kv_heads() // (world if tp else 1)) * cfg.hd * (T_prof + 1) * es
        dominant = "persistent decode-step kernel (all linears, RoPE, cache append and attention of a decode step in one launch)"
    hbm, which = peaks()
    achieved = (lin_bytes * n_prof / 1e9) / (lin_ms / 1e3) if lin_ms > 0 else 0.0
    traffic = None
    traffic_path = os.path.join(ROOT, "profiles", "gemv_traffic.json")
    if os.path.exists(traffic_path):
        with open(traffic_path) as fh:
            tj = json.load(fh)
        # dram bytes per algorithmic byte measured by ncu on the same kernel, scaled to one launch of this workload
        ratio = tj.get("dram_bytes_per_algorithmic_byte", 0)
        if gpt.DecodePath() == 2:
            ratio = tj.get("owner_kernel", {}).get("dram_bytes_per_algorithmic_byte", ratio)
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
                   "parallelism": ("tensor-parallel x%d (heads and FFN sharded; the two sums per layer are exchanged inside the decode-step kernel)" % world) if tp else "batch-sharded replicas x%d" % world,
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
        "prefill": {"tokens_per_s": seqs * S / (prefill_ms / 1e3), "ms": prefill_ms, "first_call_ms": first_prefill_ms,
                    "tflops": prefill_flops(cfg, seqs, S) / 1e12 / (prefill_ms / 1e3) / (1 if tp else world)},
        "kernel_classes_ms_per_step": {k: v[0] / n_prof for k, v in prof.items()},
        "host_wall_ms_per_step": 1e3 * t_wall / K,
        "decode_path": {0: "one launch per operation", 1: "stream-K persistent kernel", 2: "owner-partitioned persistent kernel"}.get(gpt.DecodePath()),
    }
    if prof["attention"][1] > 0:
        # the KV cache read by the decode attention of one step against the time of its launches
        kv = B * cfg.L * 2 * (cfg.kv_heads() // (world if tp else 1)) * cfg.hd * T_prof * es
        a_ms = prof["attention"][0] / n_prof
        line["attention"] = {"kv_bytes_per_step": kv, "ms_per_step": a_ms, "kv_gbs": kv / 1e9 / (a_ms / 1e3),
                             "frac_of_hbm_peak": kv / 1e9 / (a_ms / 1e3) / hbm}

    # ---- outside the timed region: the benchmarked engine against an independent one fed the same ids
    if not args.no_parity_check:
        checker = rank == 0 or not tp
        ref = per_operation_engine(cfg, local, B, S + n_check + 8, SEED) if checker else None
        barrier()   # the checker is built before the first collective step, so no rank waits inside a kernel for it
        tol = 2e-2 if cfg.dtype == "float16" else 1e-3
        pc = parity_check(gpt, ref, prompt, opts, n_check, tol)
        if ref is not None:
            ref.close()
        pc["max_rel_logit_err"] = max_over_ranks(pc["max_rel_logit_err"]) if not tp else pc["max_rel_logit_err"]
        pc["ok"] = bool(pc["max_rel_logit_err"] <= tol)
        line["parity_check"] = pc

    if world == 1 and not tp and S >= 16 and S <= 4096:
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
    gpt.close()
    if tp and not args.no_secondary:
        # beside the sharded model: the same GPUs as N independent replicas (the reference's own multi-device form), each
        # decoding its own sequences; no collective on the data path
        rep_gpt = GPT(cfg, device_id=local, max_batch=B, max_tokens=max_tokens)
        rep_gpt.FillSynthetic(SEED, 0.02, 0.0)
        rep_prompt = prompt_ids(SEED + rank, B, S, cfg.V)
        rep_opts = make_options(strat, topP, max_tokens, SEED, rank * B)
        rep_gpt.Prefill(rep_prompt, rep_opts)
        rep_gpt.Decode(W, rep_opts)
        barrier()
        rep_gpt.Decode(K, rep_opts)
        rep_ms, _ = rep_gpt.LastTiming()
        rep_ms = max_over_ranks(rep_ms)
        rep_gpt.close()
        line["replicas"] = {"value": world * B * K / (rep_ms / 1e3), "unit": "tokens/s", "ms_per_step": rep_ms / K, "scaling": "weak",
                            "note": "%d independent engines, one per GPU, %d sequence(s) each" % (world, B)}
    if world == 1 and args.workload == "c5_b1" and not args.no_secondary:
        # the other figures the metric names, each on its own engine (outside the headline timed region)
        line["secondary"] = {
            "c5_b64": measure_secondary(local, "c5_llama7b_fp16", 64, 512, "topp", 0.95, want_prefill=True),
            "c3_b32": measure_secondary(local, "c3_llama1b_fp16", 32, 1024, "greedy", 1.0),
            "c5_b4": measure_secondary(local, "c5_llama7b_fp16", 4, 512, "topp", 0.95),
            "c4_b4": measure_secondary(local, "c4_llama1b_longctx_fp16", 4, 16384, "greedy", 1.0, want_prefill=True),
            "c5_mixed_b4": measure_mixed_batch(local, "c5_llama7b_fp16", [512, 384, 256, 128]),
        }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import cpu_oracle as O
        thr = O.max_threads()
        smp = CpuSample(cfg, thr)
        v_all = smp.measure(4)
        v_one = CpuSample(cfg, 1).measure(2)
        line["cpu_baseline"] = {
            "value": v_all, "unit": "tokens/s", "cores": thr, "kind": "port", "value_1_thread": v_one,
            "sample": "CPU oracle (restatement of the reference's TensorSharp.Cpu fp32 path, reference-style realloc+copy KV cache), B=1: "
                      "%s, timed over 4 decode steps; the 1-thread figure matches the reference's single-threaded managed SGEMM" % smp.describe()}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if "parity_check" in line and not line["parity_check"]["ok"]:
        sys.exit("bench: parity check failed: logits differ by %.3g relative (tolerance %g)" %
                 (line["parity_check"]["max_rel_logit_err"], line["parity_check"]["tolerance"]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c5_b1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity-check", action="store_true")
    ap.add_argument("--no-secondary", action="store_true")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "replicas", "tp"],
                    help="N > 1: 'tp' = one model sharded over the GPUs, the two sums per layer exchanged over NVLink (strong "
                         "scaling); 'replicas' = batch-sharded independent sequences (weak scaling); 'auto' = tp for the "
                         "7B-class workloads (c5_*), replicas otherwise")
    args = ap.parse_args()
    # stdout carries the ONE JSON line: whatever NCCL has to say (its version banner, INFO lines) goes to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
