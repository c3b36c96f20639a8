"""Top-P sort-and-sample on the device must return the SAME index as the reference's host loop
(ComputeGraphTensor.TopPSample, ComputeGraphTensor.cs:2305-2403, restated in the oracle) given identical
probabilities and uniform draws — bit-exact, including the order of equal weights, the fp32 rounding of the
sequential prefix sum, the inclusive stop at acc >= topP, dropped w <= 0 entries and the repeat penalty."""
import numpy as np
import pytest
import torch

from seq2seqsharp_b200.ops import Ops

pytestmark = pytest.mark.gpu


def run(probs, topP, penalty, seqs, u):
    out = Ops.TopPSample(torch.from_numpy(probs).cuda(), topP, penalty, seqs, torch.from_numpy(np.asarray(u, np.float32)))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def softmax64(z):
    e = np.exp(z - z.max(-1, keepdims=True))
    return (e / e.sum(-1, keepdims=True)).astype(np.float32)


def test_hand_cases(cuda, oracle):
    p = np.array([[0.1, 0.4, 0.2, 0.3]], dtype=np.float32)
    assert run(p, 0.65, 0.0, None, [0.5])[0] == 1
    assert run(p, 0.65, 0.0, None, [0.6])[0] == 3
    q = np.array([[0.25, 0.25, 0.25, 0.25]] * 4, dtype=np.float32)
    assert list(run(q, 1.0, 0.0, None, [0.1, 0.3, 0.6, 0.9])) == [0, 1, 2, 3]
    r = np.array([[0.6 - 1.0, 0.3, 0.1, 0.0]], dtype=np.float32)
    assert run(r, 1.0, 0.0, None, [0.0])[0] == 1
    assert run(p, 0.2, 2.0, [[5, 1, 2, 1]], [0.0])[0] == 3
    assert run(np.zeros((1, 4), np.float32), 0.9, 2.0, None, [0.3])[0] == 0


@pytest.mark.parametrize("V", [97, 1000, 32000, 50257])
@pytest.mark.parametrize("kind", ["near_uniform", "peaky", "ties", "blocked"])
def test_bit_exact_vs_oracle(cuda, oracle, V, kind):
    rng = np.random.default_rng(V * 7 + len(kind))
    B = 6
    if kind == "near_uniform":      # N(0, 0.02)-weight models give almost flat distributions: nucleus ~ 0.9 V
        p = softmax64(rng.standard_normal((B, V)) * 0.05)
    elif kind == "peaky":
        p = softmax64(rng.standard_normal((B, V)) * 6.0)
    elif kind == "ties":            # many exactly equal probabilities: order inside a group = ascending index
        p = softmax64(np.round(rng.standard_normal((B, V)) * 2.0))
    else:
        p = softmax64(rng.standard_normal((B, V)) * 1.5)
        p[:, rng.integers(0, V, 5)] += np.float32(-1.0)
        p[:, 0] += np.float32(-1.0)
    seqs = [list(map(int, rng.integers(0, V, rng.integers(1, 60)))) for _ in range(B)]
    for topP, pen in [(0.9, 2.0), (0.95, 2.0), (1.0, 0.0), (0.5, 1.3)]:
        u = rng.random(B).astype(np.float32)
        exp = oracle.topp(p, topP, pen, seqs, u)
        got = run(p, topP, pen, seqs, u)
        np.testing.assert_array_equal(got, exp, err_msg="%s V=%d topP=%g penalty=%g" % (kind, V, topP, pen))
    # no history at all
    u = rng.random(B).astype(np.float32)
    np.testing.assert_array_equal(run(p, 0.9, 2.0, None, u), oracle.topp(p, 0.9, 2.0, None, u))


def test_extreme_draws_and_determinism(cuda, oracle):
    rng = np.random.default_rng(3)
    p = softmax64(rng.standard_normal((4, 32000)) * 0.05)
    for u in ([0.0] * 4, [np.float32(1.0) - np.float32(2 ** -24)] * 4, [1.0] * 4):
        np.testing.assert_array_equal(run(p, 0.9, 0.0, None, u), oracle.topp(p, 0.9, 0.0, None, np.asarray(u, np.float32)))
    a = run(p, 0.9, 0.0, None, [0.3, 0.5, 0.7, 0.9])
    for _ in range(3):
        np.testing.assert_array_equal(run(p, 0.9, 0.0, None, [0.3, 0.5, 0.7, 0.9]), a)
