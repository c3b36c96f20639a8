"""Mixture-of-experts decoder layers (Seq2SeqSharp/Layers/MoEFeedForward.cs, Networks/GPTDecoder.cs:114-123: layers 2.. of a
model with expertNum > 1) against the CPU oracle: prompt and token loop, logits at every step, ids by the recorded-tie
rule of tests/test_gpt_gpu.py.  fp32 models are compared at 1e-3; the router works on logits that the reference rounds to
multiples of 2^-7 (its constant -65000 mask), so equal router probabilities are common and the TopK tie rule matters."""
import numpy as np
import pytest

from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, DecodingOptions, DecodingStrategyEnums as DS, GPT, GPTConfig,
                                   MultiHeadAttentionTypeEnums as M, NormEnums as Nm, PositionEmbeddingEnums as P, synthetic_weights)
from seq2seqsharp_b200.synthetic import prompt_ids
from tests.test_gpt_gpu import compare_run, rel_err, tol_for

pytestmark = pytest.mark.gpu

CFGS = [
    GPTConfig(name="moe_e4_k2_relu", L=4, d=128, H=4, hd=32, F=256, V=503, norm=Nm.LayerNorm, act=A.ReLU, pe=P.RoPE, attn=M.MHA, dtype="float32",
              expertNum=4, expertsPerTokenFactor=2),
    GPTConfig(name="moe_e8_k1_silu_gqa", L=3, d=256, H=8, Hkv=2, hd=32, F=512, V=499, norm=Nm.RMSNorm, act=A.SiLU, pe=P.RoPE, attn=M.GQA,
              dtype="float32", expertNum=8, expertsPerTokenFactor=1),
    GPTConfig(name="moe_e5_k3_leaky_ape", L=3, d=64, H=2, hd=32, F=128, V=211, norm=Nm.LayerNorm, act=A.LeakyReLU, pe=P.APE, attn=M.MHA,
              dtype="float32", expertNum=5, expertsPerTokenFactor=3),
]
MAX_TOK = 40


@pytest.mark.parametrize("cfg", CFGS, ids=[c.name for c in CFGS])
@pytest.mark.parametrize("B,strat", [(1, DS.GreedySearch), (3, DS.Sampling)], ids=["b1_greedy", "b3_topp"])
def test_moe_token_loop_matches_oracle(cuda, oracle, cfg, B, strat):
    S, n_new = 9, 12
    w = synthetic_weights(cfg, 6, std=0.06, bias_std=0.03, max_pos=MAX_TOK + 2)
    assert any(".MoEFFN_" in k for k in w) and not any(k.startswith("GPTDecoder.PosFFN_2.") for k in w)
    prompt = prompt_ids(8, B, S, cfg.V)
    opts = DecodingOptions(MaxTgtSentLength=S + n_new, DecodingStrategy=strat, TopP=0.9, BlockedTokens=[0], Seed=2)
    orc = oracle.OracleGPT(cfg, w, max_pos=MAX_TOK + 2)
    steps = {}
    o_ids = orc.generate(prompt, opts, uniforms=lambda st, b: oracle.philox_uniform(opts.Seed, opts.SeqBase + b, st), stop_on_eos=False,
                         record=lambda st, lg, p, n: steps.update({st: (lg.copy(), p.copy(), n.copy())}))
    g = GPT(cfg, max_batch=B, max_tokens=MAX_TOK)
    g.LoadWeights(w)
    d_ids = np.zeros((B, n_new), dtype=np.int32)
    d_logits = []
    d_ids[:, 0] = g.Prefill(prompt, opts)
    d_logits.append(g.Logits())
    for i in range(1, n_new):
        d_ids[:, i] = g.Decode(1, opts)[:, 0]
        d_logits.append(g.Logits())
    assert g.DecodePath() == 0
    ties = compare_run(oracle, cfg, o_ids, steps, d_ids, d_logits, opts, prompt)
    print("%s B=%d: ties %s" % (cfg.name, B, ties))
    # the graph-replayed loop gives the same ids, and nothing wrote out of bounds
    g.Reset()
    first = g.Prefill(prompt, opts)
    np.testing.assert_array_equal(np.concatenate([first[:, None], g.Decode(n_new - 1, opts)], axis=1), d_ids)
    g.CheckGuards()
    g.close()


def test_moe_fp16_runs_and_is_reproducible(cuda):
    """fp16 weights: the router works in fp32 (in fp16 the reference's -65000 mask would round every router logit to the
    same value); checked here: finite logits, run-to-run equality, guards."""
    cfg = GPTConfig(name="moe_fp16", L=4, d=256, H=8, Hkv=4, hd=32, F=512, V=1009, norm=Nm.RMSNorm, act=A.SiLU, pe=P.RoPE, attn=M.GQA,
                    dtype="float16", expertNum=6, expertsPerTokenFactor=2)
    g = GPT(cfg, max_batch=2, max_tokens=48)
    g.FillSynthetic(5, 0.05, 0.02)
    opts = DecodingOptions(MaxTgtSentLength=48, BlockedTokens=[0])
    prompt = prompt_ids(2, 2, 17, cfg.V)
    a = np.concatenate([g.Prefill(prompt, opts)[:, None], g.Decode(10, opts)], axis=1)
    lg = g.Logits(want_probs=False)[0]
    assert np.isfinite(lg).all()
    g.Reset()
    b = np.concatenate([g.Prefill(prompt, opts)[:, None], g.Decode(10, opts)], axis=1)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(lg, g.Logits(want_probs=False)[0])
    g.CheckGuards()
    g.close()


def test_moe_config_errors(cuda):
    base = dict(L=3, d=64, H=2, hd=32, F=128, V=101, dtype="float32")
    from seq2seqsharp_b200._native import TSB200Error
    with pytest.raises(TSB200Error, match="experts"):
        GPT(GPTConfig(expertNum=4, expertsPerTokenFactor=5, **base), max_batch=1, max_tokens=8)
    g = GPT(GPTConfig(expertNum=4, expertsPerTokenFactor=1, **base), max_batch=1, max_tokens=8)
    with pytest.raises(TSB200Error, match="mixture-of-experts layer"):
        g.LoadWeights({"GPTDecoder.PosFFN_2.feedForwardLayer1.m_Whd": np.zeros((64, 128), dtype=np.float32)})
    with pytest.raises(TSB200Error, match="not a mixture-of-experts layer"):
        g.LoadWeights({"GPTDecoder.MoEFFN_0.m_Router": np.zeros((64, 4), dtype=np.float32)})
    g.close()
