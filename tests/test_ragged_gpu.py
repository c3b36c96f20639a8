"""Sequences with their own cache lengths: prompts of different lengths in one prefill, a slot of the batch parked,
refilled and restored while the others run on, and the per-sequence stop rule.

The reference pads the prompts of a batch to one length and masks the pads (BuildInTokens.PadSentences +
BuildSelfTriMask, Applications/Decoder.cs:656,687-692); the engine keeps a cache length, position, Philox step and stop
flag per sequence instead.  The bar: every sequence of a mixed batch behaves exactly as the oracle run on that sequence
ALONE (logits within the dtype's tolerance at every step, ids by the recorded-tie rule of tests/test_gpt_gpu.py, top-p
choices bit-exact on the device's own probabilities with the uniforms of the Philox stream (seed, seq_base + b))."""
import dataclasses

import numpy as np
import pytest

from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, DecodingOptions, DecodingStrategyEnums as DS, GPT, GPTConfig,
                                   MultiHeadAttentionTypeEnums as M, NormEnums as Nm, PositionEmbeddingEnums as P,
                                   synthetic_weights)
from seq2seqsharp_b200.synthetic import prompt_ids
from tests.test_gpt_gpu import compare_run, rel_err, tol_for

pytestmark = pytest.mark.gpu

CFGS = [
    GPTConfig(name="mha_ape_fp32", L=2, d=128, H=4, hd=32, F=256, V=997, norm=Nm.LayerNorm, act=A.ReLU, pe=P.APE, attn=M.MHA, dtype="float32"),
    GPTConfig(name="gqa_rope_fp16", L=3, d=512, H=8, Hkv=2, hd=64, F=1024, V=2003, norm=Nm.RMSNorm, act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16"),
]
LENS = [19, 7, 12, 1]
N_NEW = 10
MAX_TOK = 64
MAX_POS = MAX_TOK + 2   # rows of the position table the engine expects for this capacity


def _prompts(cfg, seed=21):
    full = prompt_ids(seed, len(LENS), max(LENS), cfg.V)
    return [list(map(int, full[b, :n])) for b, n in enumerate(LENS)]


def _opts(strat, n_total=MAX_TOK):
    return DecodingOptions(MaxTgtSentLength=n_total, DecodingStrategy=strat, TopP=0.9, RepeatPenalty=2.0, BlockedTokens=[0], Seed=5)


def _oracle_alone(oracle, cfg, w, prompt, opts, b, n_new):
    """The oracle on ONE sequence: ids [1, n_new], per-step (logits, probs, ids); sequence b draws from stream seq_base + b."""
    o = dataclasses.replace(opts, MaxTgtSentLength=len(prompt) + n_new, SeqBase=opts.SeqBase + b)
    orc = oracle.OracleGPT(cfg, w, max_pos=MAX_POS)
    steps = {}
    ids = orc.generate(np.asarray([prompt], dtype=np.int32), o, uniforms=lambda st, _b: oracle.philox_uniform(o.Seed, o.SeqBase, st),
                       stop_on_eos=False, record=lambda st, lg, p, n: steps.update({st: (lg.copy(), p.copy(), n.copy())}))
    return o, ids, steps


@pytest.mark.parametrize("cfg", CFGS, ids=[c.name for c in CFGS])
@pytest.mark.parametrize("strat", [DS.GreedySearch, DS.Sampling], ids=["greedy", "topp"])
def test_ragged_prefill_and_decode_match_oracle_sequence_by_sequence(cuda, oracle, cfg, strat):
    w = synthetic_weights(cfg, 3, std=0.05, bias_std=0.02, max_pos=MAX_POS)
    prompts = _prompts(cfg)
    opts = _opts(strat)
    B = len(prompts)
    gpt = GPT(cfg, max_batch=B, max_tokens=MAX_TOK)
    gpt.LoadWeights(w)
    ids = np.zeros((B, N_NEW), dtype=np.int32)
    logits = []
    ids[:, 0] = gpt.PrefillRagged(prompts, opts)
    logits.append(gpt.Logits())
    np.testing.assert_array_equal(gpt.CacheLengths(), LENS)
    for i in range(1, N_NEW):
        ids[:, i] = gpt.Decode(1, opts)[:, 0]
        logits.append(gpt.Logits())
    assert gpt.DecodePath() == 0   # sequences of different lengths: one launch per operation
    np.testing.assert_array_equal(gpt.CacheLengths(), np.array(LENS) + N_NEW - 1)
    for b, prompt in enumerate(prompts):
        o, o_ids, steps = _oracle_alone(oracle, cfg, w, prompt, opts, b, N_NEW)
        d_logits = [(lg[b:b + 1], pr[b:b + 1]) for lg, pr in logits]
        ties = compare_run(oracle, cfg, o_ids, steps, ids[b:b + 1], d_logits, o, np.asarray([prompt], dtype=np.int32))
        print("%s seq %d (len %d): ties %s" % (cfg.name, b, len(prompt), ties))
    # the graph-replayed loop (ids fed back on the device) gives the same ids
    gpt.Reset()
    first = gpt.PrefillRagged(prompts, opts)
    rest = gpt.Decode(N_NEW - 1, opts)
    np.testing.assert_array_equal(np.concatenate([first[:, None], rest], axis=1), ids)
    # and so does the host-buffer step
    gpt.Reset()
    last = gpt.PrefillRagged(prompts, opts)
    for i in range(1, N_NEW):
        last = gpt.StepHost(last, opts)
        np.testing.assert_array_equal(last, ids[:, i])
    # equal lengths given as "ragged" are the ordinary prefill
    gpt.Reset()
    eq = prompt_ids(4, 2, 9, cfg.V)
    a = gpt.PrefillRagged([list(r) for r in eq], opts)
    la = gpt.Logits(want_probs=False)[0]
    gpt.Reset()
    np.testing.assert_array_equal(a, gpt.Prefill(eq, opts))
    np.testing.assert_array_equal(la, gpt.Logits(want_probs=False)[0])
    gpt.close()


@pytest.mark.parametrize("cfg", CFGS, ids=[c.name for c in CFGS])
def test_slot_is_parked_refilled_and_restored_while_the_others_run_on(cuda, oracle, cfg):
    w = synthetic_weights(cfg, 3, std=0.05, bias_std=0.02, max_pos=MAX_POS)
    prompts = _prompts(cfg)[:3]
    opts = _opts(DS.Sampling)
    B = len(prompts)
    n_a, n_b, n_c = 4, 5, 3

    def fresh():
        g = GPT(cfg, max_batch=B, max_tokens=MAX_TOK)
        g.LoadWeights(w)
        return g

    # the undisturbed run
    ref = fresh()
    r_ids = np.concatenate([ref.PrefillRagged(prompts, opts)[:, None], ref.Decode(n_a + n_b + n_c - 1, opts)], axis=1)
    ref.close()

    g = fresh()
    ids_a = np.concatenate([g.PrefillRagged(prompts, opts)[:, None], g.Decode(n_a - 1, opts)], axis=1)
    np.testing.assert_array_equal(ids_a, r_ids[:, :n_a])
    # sequence 1 leaves: park it, start another request in its place (reset + prompt in two pieces)
    snap = g.SlotSnapshot(1)
    assert snap.B == 1 and snap.T == LENS[1] + n_a - 1
    new_prompt = list(map(int, prompt_ids(77, 1, 11, cfg.V)[0]))
    g.SlotReset(1)
    # RoPE models take the prompt in two pieces (the id sampled after the head is discarded by the next piece).  With the
    # reference's absolute position table a cached call adds rows [0, S) to its S new tokens whatever is cached
    # (PositionEmbedding.cs:30-33, Decoder.cs:674-677), so there a two-piece prompt is a different computation.
    pieces = 2 if cfg.pe == P.RoPE else 1
    if pieces == 2:
        g.SlotExtend(1, new_prompt[:6], opts)
        first_new = g.SlotExtend(1, new_prompt[6:], opts)
    else:
        first_new = g.SlotExtend(1, new_prompt, opts)
    lens = g.CacheLengths()
    assert lens[1] == len(new_prompt) and lens[0] == LENS[0] + n_a - 1 and lens[2] == LENS[2] + n_a - 1
    logits_new = [g.Logits()]
    ids_b = np.zeros((B, n_b), dtype=np.int32)
    for i in range(n_b):
        ids_b[:, i] = g.Decode(1, opts)[:, 0]
        logits_new.append(g.Logits())
    # the others never noticed
    np.testing.assert_array_equal(ids_b[[0, 2]], r_ids[[0, 2], n_a:n_a + n_b])
    # the newcomer behaves like the oracle on that prompt alone.  Its Philox stream is (seed, seq_base + 1); a head
    # piece consumes step 0, so the full prompt's first id is then drawn at step 1: compare from the oracle's
    # distribution with the device's own rule instead of the oracle's ids
    o, o_ids, steps = _oracle_alone(oracle, cfg, w, new_prompt, opts, 1, n_b + 1)
    tol = tol_for(cfg)
    assert rel_err(logits_new[0][0][1], steps[0][0][0]) <= tol
    hist = list(new_prompt)
    new_ids = [first_new] + [int(x) for x in ids_b[1]]
    for i, nid in enumerate(new_ids):
        pd = logits_new[i][1][1:2]
        u = np.array([oracle.philox_uniform(opts.Seed, opts.SeqBase + 1, i + pieces - 1)], dtype=np.float32)
        want = oracle.topp(pd, opts.TopP, opts.RepeatPenalty, [hist], u)
        assert nid == int(want[0]), "newcomer step %d" % i
        hist.append(nid)
    # sequence 1 comes back: it continues exactly where it was parked
    g.SlotRestore(snap, 1)
    snap.close()
    ids_c = g.Decode(n_c, opts)
    np.testing.assert_array_equal(ids_c[1], r_ids[1, n_a:n_a + n_c])
    np.testing.assert_array_equal(ids_c[[0, 2]], r_ids[[0, 2], n_a + n_b:n_a + n_b + n_c])
    g.close()


def test_sequences_stop_one_by_one(cuda):
    """With stop_on_eos a sequence whose previous id was </s> (0) stands still: it emits 0 and neither its cache nor its
    history advance.  A head bias that makes 0 the argmax everywhere ends every sequence at its first token."""
    cfg = CFGS[0]
    w = synthetic_weights(cfg, 3, std=0.05, bias_std=0.02, max_pos=MAX_POS)
    w = dict(w)
    hb = np.array(w["FeedForward_Decoder_0.m_Bd"], dtype=np.float32).copy()
    hb.reshape(-1)[0] = 50.0
    w["FeedForward_Decoder_0.m_Bd"] = hb
    prompts = _prompts(cfg)
    opts = DecodingOptions(MaxTgtSentLength=MAX_TOK, DecodingStrategy=DS.GreedySearch)
    g = GPT(cfg, max_batch=len(prompts), max_tokens=MAX_TOK)
    g.LoadWeights(w)
    first = g.PrefillRagged(prompts, opts)
    np.testing.assert_array_equal(first, 0)
    out = g.Decode(6, opts, stop_on_eos=True)
    assert out.shape[1] == 1 and (out == 0).all()          # every sequence had ended: the loop stops after one step
    np.testing.assert_array_equal(g.CacheLengths(), LENS)  # and nothing advanced
    # without the stop rule the same call runs on
    out = g.Decode(3, opts, stop_on_eos=False)
    assert out.shape[1] == 3
    np.testing.assert_array_equal(g.CacheLengths(), np.array(LENS) + 3)
    g.close()


def test_ragged_errors(cuda):
    cfg = CFGS[0]
    g = GPT(cfg, max_batch=2, max_tokens=32)
    g.FillSynthetic(1, 0.05, 0.02)
    opts = DecodingOptions(MaxTgtSentLength=32, BlockedTokens=[0])
    with pytest.raises(RuntimeError, match="sequence index"):
        g.SlotReset(1)                      # slot 1 before slot 0 exists
    g.PrefillRagged([[5, 6, 7], [8]], opts)
    with pytest.raises(RuntimeError, match="different lengths"):
        g.CacheSnapshot()
    with pytest.raises(RuntimeError, match="different lengths"):
        g.Extend(np.array([[1], [2]], dtype=np.int32), opts)
    with pytest.raises(RuntimeError, match="sequence index"):
        g.SlotExtend(2, [1, 2], opts)       # capacity is two sequences
    with pytest.raises(RuntimeError, match="OOM"):
        g.SlotExtend(0, list(range(1, 40)), opts)
    g.close()
