"""Out-of-bounds writes without a sanitizer: every device buffer of the engine lies between two guard regions, and the host
checks them after sweeps over tiny shapes (where an index error reaches a neighbouring buffer soonest) and over the
shapes of the other GPU tests.  Each run is also compared with the CPU oracle, and repeated for bitwise equality."""
import itertools

import numpy as np
import pytest

from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, DecodingOptions, DecodingStrategyEnums as DS, GPT, GPTConfig,
                                   MultiHeadAttentionTypeEnums as M, NormEnums as Nm, PositionEmbeddingEnums as P,
                                   synthetic_weights)
from seq2seqsharp_b200.synthetic import prompt_ids
from tests.test_gpt_gpu import rel_err, tol_for

pytestmark = pytest.mark.gpu


def _tiny_configs():
    out = []
    for dtype, (norm, act, pe, attn, hkv) in itertools.product(
            ("float32", "float16"),
            ((Nm.LayerNorm, A.ReLU, P.APE, M.MHA, 0), (Nm.RMSNorm, A.SwiGLU, P.RoPE, M.GQA, 2), (Nm.RMSNorm, A.SiLU, P.RoPE, M.GQA, 1))):
        out.append(GPTConfig(name="tiny_%s_%s" % (dtype, attn.name + str(hkv)), L=2, d=64, H=4, Hkv=hkv, hd=16, F=96, V=97, norm=norm, act=act,
                             pe=pe, attn=attn, dtype=dtype))
    return out


@pytest.mark.parametrize("cfg", _tiny_configs(), ids=lambda c: c.name)
def test_tiny_shapes_leave_every_guard_intact(cuda, oracle, cfg, monkeypatch):
    max_tok = 12
    w = synthetic_weights(cfg, 2, std=0.08, bias_std=0.02, max_pos=max_tok + 2)
    tol = tol_for(cfg)
    for owner, B, S, strat in itertools.product(("1", "0"), (1, 2, 3, 5), (1, 2, 5), (DS.GreedySearch, DS.Sampling)):
        monkeypatch.setenv("TSB200_OWNER", owner)
        monkeypatch.setenv("TSB200_OWNER_MAXB", "4")
        monkeypatch.setenv("TSB200_STACK_MAXB", "4")
        opts = DecodingOptions(MaxTgtSentLength=max_tok, DecodingStrategy=strat, TopP=0.8, BlockedTokens=[0], Seed=1)
        prompt = prompt_ids(3 + B + S, B, S, cfg.V)
        g = GPT(cfg, max_batch=B, max_tokens=max_tok)
        g.LoadWeights(w)
        first = g.Prefill(prompt, opts)
        lg = g.Logits(want_probs=False)[0]
        # the oracle's logits for the prompt (every sequence alone would give the same: equal lengths)
        orc = oracle.OracleGPT(cfg, w, max_pos=max_tok + 2)
        steps = {}
        orc.generate(prompt, DecodingOptions(MaxTgtSentLength=S + 1, DecodingStrategy=DS.GreedySearch, BlockedTokens=[0]),
                     stop_on_eos=False, record=lambda st, l, p, n: steps.update({st: l.copy()}))
        assert rel_err(lg, steps[0]) <= tol, (cfg.name, owner, B, S)
        ids = g.Decode(max_tok - S - 1, opts)        # up to the last cache position
        g.CheckGuards()
        # again, bitwise
        g.Reset()
        np.testing.assert_array_equal(g.Prefill(prompt, opts), first)
        np.testing.assert_array_equal(g.Decode(max_tok - S - 1, opts), ids)
        # mixed lengths and a refilled slot on the same engine
        if B >= 2:
            g.Reset()
            g.PrefillRagged([list(map(int, prompt[b, :max(1, S - b)])) for b in range(B)], opts)
            g.Decode(2, opts)
            snap = g.SlotSnapshot(0)
            g.SlotReset(0)
            g.SlotExtend(0, [5, 6, 7], opts)
            g.Decode(1, opts)
            g.SlotRestore(snap, 0)
            snap.close()
            g.Decode(1, opts)
        g.CheckGuards()
        g.close()


def test_guards_of_a_wide_model_after_every_decode_path(cuda, monkeypatch):
    """The 7B-class layer geometry (two layers) through both persistent kernels, per-operation launches, the tcgen05
    streaming GEMM (64 rows) and a prefill long enough for the tensor-core GEMM and attention."""
    from seq2seqsharp_b200.configs import CONFIGS
    import dataclasses
    cfg = dataclasses.replace(CONFIGS["c5_llama7b_fp16"], L=2, V=4096)
    monkeypatch.setenv("TSB200_OWNER_MAXB", "1")    # the persistent kernels are opt-in on one GPU
    monkeypatch.setenv("TSB200_STACK_MAXB", "2")
    for owner, B in (("1", 1), ("0", 1), ("0", 2), ("1", 4), ("1", 64)):
        monkeypatch.setenv("TSB200_OWNER", owner)
        g = GPT(cfg, max_batch=B, max_tokens=160)
        g.FillSynthetic(3, 0.02, 0.01)
        opts = DecodingOptions(MaxTgtSentLength=160, DecodingStrategy=DS.Sampling, TopP=0.9, BlockedTokens=[0])
        g.Prefill(prompt_ids(1, B, 130, cfg.V), opts)
        g.Decode(8, opts)
        g.CheckGuards()
        g.close()
