"""CPU tests that pin the oracle (no GPU).

Pins used:
  * the input vectors of the reference's backend-comparison tests
    (Tests/Seq2SeqSharp.Tests/GgmlOpsComparison_Tests.cs:419-590: softmax, addmm, addmmbatch, argmax, LayerNorm,
    RMSNorm) with closed-form expectations evaluated in float64, at that suite's tolerance 1e-4 (:24);
  * the identity pinned by ComputeGraph_Tests.TestLogSoftmax (ComputeGraph_Tests.cs: LogSoftmax == log(Softmax), 4
    decimals);
  * the published Philox4x32-10 known-answer vectors (Random123 kat_vectors);
  * the NumPy twin of the restatement (independent code path) on whole decode steps;
  * the committed golden fixtures under tests/golden/ (regenerate with tests/golden/make_golden.py).
"""
import dataclasses
import os

import numpy as np
import pytest

from seq2seqsharp_b200 import configs
from seq2seqsharp_b200.gpt import (ActivateFuncEnums, DecodingOptions, DecodingStrategyEnums, GPTConfig,
                                   MultiHeadAttentionTypeEnums, NormEnums, PositionEmbeddingEnums, synthetic_weights)
from seq2seqsharp_b200.synthetic import fnv1a64, prompt_ids, synth

TOL = 1e-4  # GgmlOpsComparison_Tests.cs:24


def test_softmax_reference_vectors(oracle):
    vals = np.array([1, 2, 3, 4, 5, 6, 7, 8], dtype=np.float32).reshape(2, 4)  # GgmlOpsComparison_Tests.cs:423
    e = np.exp(vals.astype(np.float64) - vals.max(1, keepdims=True))
    np.testing.assert_allclose(oracle.softmax(vals), e / e.sum(1, keepdims=True), atol=TOL)
    # non-contiguous variant (:433): a [4,2] tensor viewed transposed
    v = np.array([1, 2, 3, 4, 5, 6, 7, 8], dtype=np.float32).reshape(4, 2).T
    e = np.exp(v.astype(np.float64) - v.max(1, keepdims=True))
    np.testing.assert_allclose(oracle.softmax(np.ascontiguousarray(v)), e / e.sum(1, keepdims=True), atol=TOL)


def test_logsoftmax_identity(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((8, 100)).astype(np.float32)
    lse = np.log(np.exp(x.astype(np.float64) - x.max(1, keepdims=True)).sum(1, keepdims=True)) + x.max(1, keepdims=True)
    np.testing.assert_allclose(np.log(oracle.softmax(x)), x - lse, atol=1e-4)


def test_addmm_reference_vectors(oracle):
    m1 = np.arange(1, 9, dtype=np.float32).reshape(2, 4)    # GgmlOpsComparison_Tests.cs:443
    m2 = np.arange(1, 13, dtype=np.float32).reshape(4, 3)   # :444
    out = oracle.addmm(0.0, np.zeros((2, 3), np.float32), 1.0, m1, m2)
    np.testing.assert_allclose(out, [[70, 80, 90], [158, 184, 210]], atol=TOL)
    # transposed-view variant (:455): aBase [4,2] = {1,5,2,6,3,7,4,8} transposed gives the same m1
    a = np.array([1, 5, 2, 6, 3, 7, 4, 8], dtype=np.float32).reshape(4, 2).T
    np.testing.assert_allclose(oracle.addmm(0.0, np.zeros((2, 3), np.float32), 1.0, np.ascontiguousarray(a), m2), out, atol=TOL)
    # batched vectors (:465-467), per batch
    b1 = np.arange(1, 13, dtype=np.float32).reshape(2, 3, 2)
    b2 = np.arange(1, 17, dtype=np.float32).reshape(2, 2, 4)
    for i in range(2):
        np.testing.assert_allclose(oracle.addmm(0.0, np.zeros((3, 4), np.float32), 1.0, b1[i], b2[i]),
                                   b1[i].astype(np.float64) @ b2[i].astype(np.float64), atol=TOL)
    # Affine semantics: bias first, beta = 1 (ComputeGraphTensor.cs:1877-1880)
    bias = np.array([[0.5, -1.0, 2.0]], dtype=np.float32)
    np.testing.assert_allclose(oracle.addmm(1.0, bias, 1.0, m1, m2), out + bias, atol=TOL)


def test_argmax_reference_vectors(oracle):
    vals = np.array([3, 1, 4, 1, 5, 9, 2, 6], dtype=np.float32).reshape(2, 4)  # GgmlOpsComparison_Tests.cs:529
    assert list(oracle.argmax(vals)) == [2, 1]
    v = np.array([3, 2, 1, 4, 5, 6, 9, 8], dtype=np.float32).reshape(4, 2).T     # :539
    assert list(oracle.argmax(np.ascontiguousarray(v))) == [3, 3]
    # first-max rule: lowest index among equal maxima (TensorApplyCPU.cs:339-360)
    assert list(oracle.argmax(np.array([[1, 7, 7, 0], [2, 2, 2, 2]], dtype=np.float32))) == [1, 0]


def test_norm_reference_vectors(oracle):
    vals = np.arange(1, 9, dtype=np.float32).reshape(2, 4)  # GgmlOpsComparison_Tests.cs:549,573
    g, b = np.ones(4, np.float32), np.zeros(4, np.float32)
    x = vals.astype(np.float64)
    ln = (x - x.mean(1, keepdims=True)) / np.sqrt(1e-5 + x.var(1, keepdims=True))
    np.testing.assert_allclose(oracle.layernorm(vals, g, b, 1e-5), ln, atol=TOL)
    rn = x / np.sqrt((x * x).mean(1, keepdims=True) + 1e-5)
    np.testing.assert_allclose(oracle.rmsnorm(vals, g, b, 1e-5), rn, atol=TOL)
    # non-contiguous inputs (:562,:586): {1,5,2,6,3,7,4,8} as [4,2] transposed is the same matrix
    v = np.ascontiguousarray(np.array([1, 5, 2, 6, 3, 7, 4, 8], dtype=np.float32).reshape(4, 2).T)
    np.testing.assert_allclose(oracle.layernorm(v, g, b, 1e-5), ln, atol=TOL)
    np.testing.assert_allclose(oracle.rmsnorm(v, g, b, 1e-5), rn, atol=TOL)
    # long rows exercise the 8-wide vector loop + scalar tail of the reference's LayerNorm
    rng = np.random.default_rng(1)
    xx = rng.standard_normal((3, 517)).astype(np.float32)
    gg, bb = rng.standard_normal(517).astype(np.float32), rng.standard_normal(517).astype(np.float32)
    x64 = xx.astype(np.float64)
    np.testing.assert_allclose(oracle.layernorm(xx, gg, bb, 1e-6),
                               gg * (x64 - x64.mean(1, keepdims=True)) / np.sqrt(1e-6 + x64.var(1, keepdims=True)) + bb, atol=2e-5)


def test_rope_matches_definition(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2 * 3 * 5, 64)).astype(np.float32)  # [B*H, S=5] rows
    out = oracle.rope(x, 5, 7)
    for j in (0, 4, 11, 29):
        m = (j % 5) + 7
        for i in (0, 1, 31):
            th = np.float32(500000.0 ** (-2.0 * i / 64)) * np.float32(m)
            c, s = np.cos(np.float64(np.float32(th))), np.sin(np.float64(np.float32(th)))
            assert abs(out[j, 2 * i] - (x[j, 2 * i] * c - x[j, 2 * i + 1] * s)) < 1e-6
            assert abs(out[j, 2 * i + 1] - (x[j, 2 * i + 1] * c + x[j, 2 * i] * s)) < 1e-6


def test_philox_known_answers(oracle):
    assert oracle.philox4x32_10([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert oracle.philox4x32_10([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert oracle.philox4x32_10([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    u = [oracle.philox_uniform(7, s, t) for s in range(4) for t in range(4)]
    assert all(0.0 <= v < 1.0 for v in u) and len(set(u)) == 16


def test_topp_semantics(oracle):
    """Hand-checked cases of ComputeGraphTensor.TopPSample (ComputeGraphTensor.cs:2305-2403)."""
    p = np.array([[0.1, 0.4, 0.2, 0.3]], dtype=np.float32)
    # order 1(.4) 3(.3) 2(.2) 0(.1); topP=0.65 -> nucleus {1,3} acc = .7; u=0.5 -> .4/.7=.571>=.5 -> 1 ; u=0.6 -> 3
    assert oracle.topp(p, 0.65, 0.0, None, [0.5])[0] == 1
    assert oracle.topp(p, 0.65, 0.0, None, [0.6])[0] == 3
    out, n, acc = oracle.topp(p, 0.65, 0.0, None, [0.6], return_details=True)
    assert n[0] == 2 and abs(acc[0] - 0.7) < 1e-6
    # equal weights keep ascending index order inside the group
    q = np.array([[0.25, 0.25, 0.25, 0.25]], dtype=np.float32)
    assert [int(oracle.topp(q, 1.0, 0.0, None, [u])[0]) for u in (0.1, 0.3, 0.6, 0.9)] == [0, 1, 2, 3]
    # w <= 0 entries are dropped (blocked tokens carry p - 1 < 0)
    r = np.array([[0.6 - 1.0, 0.3, 0.1, 0.0]], dtype=np.float32)
    assert oracle.topp(r, 1.0, 0.0, None, [0.0])[0] == 1
    # repeat penalty: id 1 last seen 1 position ago in a sequence of 4 -> w *= (1/4)^2
    seqs = [[5, 1, 2, 1]]
    assert oracle.topp(p, 0.2, 2.0, seqs, [0.0])[0] == 3     # 0.4*(1/16)=.025 drops below .3
    # nothing positive -> index 0 (zero-initialised result)
    assert oracle.topp(np.zeros((1, 4), np.float32), 0.9, 2.0, None, [0.3])[0] == 0


def test_synthetic_generator_is_stable():
    assert fnv1a64("") == 0xCBF29CE484222325 and fnv1a64("a") == 0xAF63DC4C8601EC8C  # published FNV-1a vectors
    w = synth("TgtEmbeddings", (64, 32), 20261125)
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "synthetic.npz"))
    np.testing.assert_array_equal(w, g["emb_64x32"])
    np.testing.assert_array_equal(prompt_ids(20261125, 3, 16, 32000), g["prompt_3x16"])
    big = synth("x", (200000,), 1)
    assert abs(big.std() - 0.02) < 2e-4 and abs(big.mean()) < 2e-4
    # offset addressing = slicing (any shard can be generated independently)
    np.testing.assert_array_equal(synth("x", (1000,), 1, offset=500), big[500:1500])


SMALL = [
    GPTConfig(name="mha_ln_relu_rope", L=2, d=64, H=4, hd=16, F=96, V=97, norm=NormEnums.LayerNorm,
              act=ActivateFuncEnums.ReLU, pe=PositionEmbeddingEnums.RoPE, attn=MultiHeadAttentionTypeEnums.MHA),
    GPTConfig(name="mha_ln_gelu_ape", L=2, d=64, H=4, hd=16, F=96, V=97, norm=NormEnums.LayerNorm,
              act=ActivateFuncEnums.GELU, pe=PositionEmbeddingEnums.APE, attn=MultiHeadAttentionTypeEnums.MHA),
    GPTConfig(name="gqa_rms_swiglu_rope", L=2, d=64, H=4, Hkv=2, hd=16, F=96, V=97, norm=NormEnums.RMSNorm,
              act=ActivateFuncEnums.SwiGLU, pe=PositionEmbeddingEnums.RoPE, attn=MultiHeadAttentionTypeEnums.GQA),
    GPTConfig(name="gqa_rms_silu_nope", L=1, d=64, H=4, Hkv=1, hd=16, F=96, V=97, norm=NormEnums.RMSNorm,
              act=ActivateFuncEnums.SiLU, pe=PositionEmbeddingEnums.NoPE, attn=MultiHeadAttentionTypeEnums.GQA),
]


@pytest.mark.parametrize("cfg", SMALL, ids=[c.name for c in SMALL])
@pytest.mark.parametrize("faithful", [False, True])
def test_cpp_oracle_matches_numpy_twin(oracle, cfg, faithful):
    from oracle.np_oracle import NpGPT
    w = synthetic_weights(cfg, 11, std=0.08, bias_std=0.05, max_pos=40)
    a = oracle.OracleGPT(cfg, w, max_pos=40, faithful_cache=faithful)
    b = NpGPT(cfg, w)
    ids = prompt_ids(3, 2, 6, cfg.V)
    la, pa = a.step(ids)
    lb, pb = b.step(ids)
    np.testing.assert_allclose(la, lb, rtol=0, atol=2e-5 * np.abs(lb).max())
    np.testing.assert_allclose(pa, pb, atol=1e-6)
    for t in range(4):
        nxt = oracle.argmax(pa).reshape(-1, 1)
        la, pa = a.step(nxt)
        lb, pb = b.step(nxt)
        np.testing.assert_allclose(la, lb, rtol=0, atol=2e-5 * np.abs(lb).max())


def test_oracle_threads_do_not_change_results(oracle):
    cfg = dataclasses.replace(SMALL[2], d=128, H=8, Hkv=2, F=640, V=1031)
    w = synthetic_weights(cfg, 5, std=0.05)
    ids = prompt_ids(9, 2, 5, cfg.V)
    l1, _ = oracle.OracleGPT(cfg, w, threads=1).step(ids)
    l4, _ = oracle.OracleGPT(cfg, w, threads=4).step(ids)
    np.testing.assert_array_equal(l1, l4)


def test_oracle_against_committed_goldens(oracle):
    """The committed fixtures were produced by tests/golden/make_golden.py from this oracle; a change in the oracle's
    arithmetic (or in the synthetic generator) shows up here before any GPU is involved."""
    from tests.golden.make_golden import CASES, run_case
    path = os.path.join(os.path.dirname(__file__), "golden", "gpt_goldens.npz")
    g = np.load(path)
    for case in CASES:
        res = run_case(case)
        for k, v in res.items():
            key = "%s/%s" % (case["name"], k)
            if v.dtype.kind in "iu":
                np.testing.assert_array_equal(v, g[key], err_msg=key)
            else:
                np.testing.assert_allclose(v, g[key], rtol=0, atol=1e-6 * max(1.0, float(np.abs(g[key]).max())), err_msg=key)


def test_topk_follows_the_reference_loop(oracle):
    """TensorApplyCPU.TopK / replace_smaller (TensorSharp/TensorApplyCPU.cs:1097-1146), restated literally in Python, on
    random rows and on rows full of ties (the router of a mixture-of-experts layer produces many: its logits are rounded
    to multiples of 2^-7)."""
    def ref(row, k):
        val, idx = [-1.70141e+38] * k, [-1] * k
        for i, data in enumerate(row):
            if data < val[k - 1]:
                continue
            placed = False
            for j in range(k - 2, -1, -1):
                if data > val[j]:
                    val[j + 1], idx[j + 1] = val[j], idx[j]
                else:
                    val[j + 1], idx[j + 1] = data, i
                    placed = True
                    break
            if not placed:
                val[0], idx[0] = data, i
        return val, idx

    rng = np.random.default_rng(3)
    for cols, k in ((8, 1), (8, 2), (5, 5), (64, 4), (3, 1)):
        x = rng.standard_normal((40, cols)).astype(np.float32)
        x[10:30] = np.round(x[10:30] * 2) / 2          # ties
        x[30:] = 0.125                                  # all equal
        val, idx = oracle.topk(x, k)
        for r in range(x.shape[0]):
            v, i = ref([float(t) for t in x[r]], k)
            assert list(idx[r]) == i and [float(t) for t in val[r]] == v, (cols, k, r)
    # k = 1: the LAST of equal maxima wins (data < array[0] is the only early exit)
    assert oracle.topk(np.array([[1.0, 3.0, 3.0, 2.0]], dtype=np.float32), 1)[1][0, 0] == 2
