"""Generates the golden fixtures under tests/golden/ from the CPU oracle (python -m tests.golden.make_golden).

The reference (C#) cannot run in the build environment and ships no known-answer vector for the GPT decode loop,
so these fixtures are produced by the oracle restatement: seeded weights and prompts, logits of the prefill step
and of selected decode steps, the greedy ids, and top-p ids for the seeded Philox uniforms.  They pin the oracle
against drift and give the GPU tests a second, file-based comparison that needs no oracle run.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import cpu_oracle as O  # noqa: E402
from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, DecodingOptions, DecodingStrategyEnums as DS, GPTConfig,  # noqa: E402
                                   MultiHeadAttentionTypeEnums as M, NormEnums as Nm, PositionEmbeddingEnums as P,
                                   synthetic_weights)
from seq2seqsharp_b200.synthetic import prompt_ids, synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SEED = 20261125

# Down-scaled versions of the five benchmark architectures (same switches, small dims) so the oracle runs in seconds.
CASES = [
    dict(name="c1_arch_fp32_greedy", cfg=GPTConfig(L=3, d=128, H=4, hd=32, F=256, V=997, norm=Nm.LayerNorm, act=A.ReLU,
                                                   pe=P.RoPE, attn=M.MHA, dtype="float32"),
         B=1, S=12, n_new=24, strategy=DS.GreedySearch, topP=1.0, std=0.05, bias_std=0.02),
    dict(name="c2_arch_fp16_topp", cfg=GPTConfig(L=2, d=96, H=3, hd=32, F=192, V=1009, norm=Nm.LayerNorm, act=A.GELU,
                                                 pe=P.APE, attn=M.MHA, dtype="float16"),
         B=3, S=9, n_new=16, strategy=DS.Sampling, topP=0.9, std=0.05, bias_std=0.02),
    dict(name="c3_arch_fp16_greedy", cfg=GPTConfig(L=2, d=128, H=8, Hkv=2, hd=16, F=320, V=991, norm=Nm.RMSNorm,
                                                   act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16"),
         B=2, S=17, n_new=20, strategy=DS.GreedySearch, topP=1.0, std=0.05, bias_std=0.0),
    dict(name="c5_arch_fp16_topp", cfg=GPTConfig(L=2, d=256, H=4, Hkv=2, hd=64, F=352, V=1013, norm=Nm.RMSNorm,
                                                 act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16"),
         B=2, S=8, n_new=16, strategy=DS.Sampling, topP=0.95, std=0.05, bias_std=0.02),
]


def case_inputs(case):
    cfg = case["cfg"]
    max_pos = case["S"] + case["n_new"] + 2
    w = synthetic_weights(cfg, SEED, std=case["std"], bias_std=case["bias_std"], max_pos=max_pos + 2)
    prompt = prompt_ids(SEED, case["B"], case["S"], cfg.V)
    opts = DecodingOptions(MaxTgtSentLength=case["S"] + case["n_new"], DecodingStrategy=case["strategy"], TopP=case["topP"],
                           Temperature=1.0, RepeatPenalty=2.0, BlockedTokens=[0], Seed=SEED, SeqBase=0)
    return cfg, w, prompt, opts, max_pos + 2


def run_case(case):
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    orc = O.OracleGPT(cfg, w, max_pos=max_pos)
    rec = {}

    def record(step, logits, probs, nxt):
        if step in (0, 1, case["n_new"] - 1):
            rec["logits_step%d" % step] = logits.copy()

    ids = orc.generate(prompt, opts, uniforms=lambda step, b: O.philox_uniform(SEED, b, step), stop_on_eos=False, record=record)
    rec["ids"] = ids.astype(np.int32)
    return rec


def main():
    out = {}
    for case in CASES:
        for k, v in run_case(case).items():
            out["%s/%s" % (case["name"], k)] = v
    np.savez_compressed(os.path.join(HERE, "gpt_goldens.npz"), **out)
    np.savez_compressed(os.path.join(HERE, "synthetic.npz"), emb_64x32=synth("TgtEmbeddings", (64, 32), SEED),
                        prompt_3x16=prompt_ids(SEED, 3, 16, 32000))
    print("wrote", sorted(out))


if __name__ == "__main__":
    main()
