"""GPU parity of the unfused ops (the op names OpRegistry dispatches) against the CPU oracle, through the C ABI.

Modelled on the reference's backend-vs-backend suite (Tests/Seq2SeqSharp.Tests/GgmlOpsComparison_Tests.cs): every op
runs on contiguous and, where the ABI accepts views, on transposed / expanded inputs, and must agree with the CPU
path within that suite's 1e-4 (fp32).  fp16 tensors are compared at 2e-3 against the fp32 oracle evaluated on the
rounded inputs.
"""
import numpy as np
import pytest
import torch

from seq2seqsharp_b200 import _native as N
from seq2seqsharp_b200.ops import Ops

pytestmark = pytest.mark.gpu
TOL = 1e-4


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    torch.cuda.synchronize()
    return t.float().cpu().numpy()


def test_copy_fill_views(cuda):
    vals = np.arange(1, 7, dtype=np.float32).reshape(2, 3)  # GgmlOpsComparison_Tests.cs:74-92
    src = dev(vals)
    r = torch.empty(2, 3, device=cuda)
    np.testing.assert_array_equal(host(Ops.Copy(r, src)), vals)
    rt = torch.empty(3, 2, device=cuda)
    np.testing.assert_array_equal(host(Ops.Copy(rt, src.t())), vals.T)             # transposed view as source
    re = torch.empty(4, 3, device=cuda)
    np.testing.assert_array_equal(host(Ops.Copy(re, src[:1].expand(4, 3))), np.repeat(vals[:1], 4, 0))  # stride-0 view
    np.testing.assert_array_equal(host(Ops.Fill(torch.empty(5, 7, device=cuda), 2.5)), np.full((5, 7), 2.5, np.float32))
    h = Ops.Float2Half(None, src)
    assert h.dtype == torch.float16
    np.testing.assert_array_equal(host(Ops.Half2Float(None, h)), vals)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL), (torch.float16, 2e-3)])
def test_elementwise(cuda, oracle, dtype, tol):
    rng = np.random.default_rng(0)
    a = rng.standard_normal((6, 33)).astype(np.float32)
    b = rng.standard_normal((6, 33)).astype(np.float32)
    A, B = dev(a, dtype), dev(b, dtype)
    a, b = host(A), host(B)
    np.testing.assert_allclose(host(Ops.Add(None, A, B)), a + b, atol=tol)
    np.testing.assert_allclose(host(Ops.Mul(None, A, B)), a * b, atol=tol)
    np.testing.assert_allclose(host(Ops.Mul(None, A, 3.0)), a * 3.0, atol=tol * 3)
    np.testing.assert_allclose(host(Ops.Div(None, A, 0.7)), a / np.float32(0.7), atol=tol * 2)
    np.testing.assert_allclose(host(Ops.Relu(None, A)), oracle.act(a, 0), atol=tol)
    np.testing.assert_allclose(host(Ops.SiLU(None, A)), oracle.act(a, 1), atol=tol)
    np.testing.assert_allclose(host(Ops.LeakyReLU(None, A)), oracle.act(a, 2), atol=tol)
    # broadcast of a [1, n] bias row through a stride-0 view (how Affine passes its bias: ComputeGraphTensor.cs:1877)
    np.testing.assert_allclose(host(Ops.Add(None, A, B[:1].expand(6, 33))), a + b[:1], atol=tol)
    # transposed operand
    At = dev(a.T.copy(), dtype).t()
    np.testing.assert_allclose(host(Ops.Add(None, At, B)), a + b, atol=tol)


def test_softmax(cuda, oracle):
    vals = np.arange(1, 9, dtype=np.float32).reshape(2, 4)
    np.testing.assert_allclose(host(Ops.Softmax(None, dev(vals))), oracle.softmax(vals), atol=TOL)
    v = dev(np.arange(1, 9, dtype=np.float32).reshape(4, 2)).t()                   # GgmlOpsComparison_Tests.cs:433
    np.testing.assert_allclose(host(Ops.Softmax(None, v)), oracle.softmax(np.ascontiguousarray(host(v))), atol=TOL)
    rng = np.random.default_rng(1)
    for shape in [(3, 1), (5, 50257), (2, 3, 7, 129)]:
        x = (rng.standard_normal(shape) * 4).astype(np.float32)
        out = host(Ops.Softmax(None, dev(x)))
        np.testing.assert_allclose(out, oracle.softmax(x), atol=1e-6, rtol=1e-4)
        np.testing.assert_allclose(out.sum(-1), 1.0, atol=1e-5)
    xh = dev(rng.standard_normal((4, 300)).astype(np.float32), torch.float16)
    np.testing.assert_allclose(host(Ops.Softmax(None, xh)), oracle.softmax(host(xh)), atol=2e-3)


def test_argmax(cuda, oracle):
    vals = np.array([3, 1, 4, 1, 5, 9, 2, 6], dtype=np.float32).reshape(2, 4)      # GgmlOpsComparison_Tests.cs:529
    assert list(host(Ops.Argmax(None, dev(vals), 1)).reshape(-1)) == [2, 1]
    v = dev(np.array([3, 2, 1, 4, 5, 6, 9, 8], dtype=np.float32).reshape(4, 2)).t()  # :539
    assert list(host(Ops.Argmax(None, v, 1)).reshape(-1)) == [3, 3]
    ties = np.zeros((3, 40000), dtype=np.float32)
    ties[0, [17, 39999, 20000]] = 2.0   # lowest index wins
    ties[1, :] = 1.0
    ties[2, 39999] = 5.0
    assert list(host(Ops.Argmax(None, dev(ties), 1)).reshape(-1)) == [17, 0, 39999]
    rng = np.random.default_rng(2)
    x = rng.standard_normal((7, 32000)).astype(np.float32)
    assert list(host(Ops.Argmax(None, dev(x), -1)).reshape(-1).astype(np.int32)) == list(oracle.argmax(x))
    # reduction over dim 0
    y = rng.standard_normal((50, 9)).astype(np.float32)
    assert list(host(Ops.Argmax(None, dev(y), 0)).reshape(-1).astype(np.int64)) == list(y.argmax(0))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL), (torch.float16, 4e-3)])
@pytest.mark.parametrize("cols", [4, 512, 768, 4096, 517])
def test_norms(cuda, oracle, dtype, tol, cols):
    rng = np.random.default_rng(cols)
    x = rng.standard_normal((5, cols)).astype(np.float32) * 2 + 0.3
    g = rng.standard_normal(cols).astype(np.float32)
    b = rng.standard_normal(cols).astype(np.float32)
    X, G, Bt = dev(x, dtype), dev(g, dtype), dev(b, dtype)
    x, g, b = host(X), host(G), host(Bt)
    np.testing.assert_allclose(host(Ops.LayerNorm(None, X, G, Bt, 1e-6)), oracle.layernorm(x, g, b, 1e-6), atol=tol * 4)
    np.testing.assert_allclose(host(Ops.LayerNorm(None, X, G, None, 1e-6)), oracle.layernorm(x, g, None, 1e-6), atol=tol * 4)
    np.testing.assert_allclose(host(Ops.RMSNorm(None, X, G, None, 1e-6)), oracle.rmsnorm(x, g, None, 1e-6), atol=tol * 4)
    np.testing.assert_allclose(host(Ops.RMSNorm(None, X, G, Bt, 1e-6)), oracle.rmsnorm(x, g, b, 1e-6), atol=tol * 4)


def test_norm_reference_vectors_and_row_strided_view(cuda, oracle):
    vals = np.arange(1, 9, dtype=np.float32).reshape(2, 4)                          # GgmlOpsComparison_Tests.cs:549
    g, b = np.ones(4, np.float32), np.zeros(4, np.float32)
    np.testing.assert_allclose(host(Ops.LayerNorm(None, dev(vals), dev(g), dev(b), 1e-5)), oracle.layernorm(vals, g, b, 1e-5), atol=TOL)
    np.testing.assert_allclose(host(Ops.RMSNorm(None, dev(vals), dev(g), dev(b), 1e-5)), oracle.rmsnorm(vals, g, b, 1e-5), atol=TOL)
    wide = dev(np.arange(16, dtype=np.float32).reshape(2, 8))
    view = wide[:, :4]                                                             # rows strided by 8
    np.testing.assert_allclose(host(Ops.RMSNorm(None, view, dev(g), None, 1e-5)), oracle.rmsnorm(host(view), g, None, 1e-5), atol=TOL)
    # a column-strided (transposed) view is refused with a clear error, as the reference's CUDA op requires contiguity
    with pytest.raises(N.TSB200Error):
        Ops.RMSNorm(None, dev(np.arange(8, dtype=np.float32).reshape(4, 2)).t(), dev(g), None, 1e-5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 2e-3)])
def test_rope(cuda, oracle, dtype, tol):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2 * 4 * 5, 64)).astype(np.float32)
    X = dev(x, dtype)
    x = host(X)
    for off in (0, 7, 1500):
        np.testing.assert_allclose(host(Ops.RoPE(None, X, 5, off)), oracle.rope(x, 5, off), atol=tol)
    np.testing.assert_allclose(host(Ops.RoPE(None, X, 5, 3, base=10000.0)), oracle.rope(x, 5, 3, 10000.0), atol=tol)


def test_indexselect_and_masks(cuda, oracle):
    rng = np.random.default_rng(4)
    src = rng.standard_normal((50, 24)).astype(np.float32)
    idx = np.array([3, 49, 0, -1, 7], dtype=np.float32)                             # float indices, negative = skip
    out0 = np.full((5, 24), 9.0, dtype=np.float32)
    r = dev(out0)
    Ops.IndexSelect(r, dev(src), dev(idx.reshape(-1, 1)))
    np.testing.assert_array_equal(host(r), oracle.indexselect(src, idx, out0.copy()))
    m = Ops.BuildTriMask(torch.empty(6, 6, device=cuda), 0.0, -30000.0)
    exp = np.where(np.arange(6)[None, :] <= np.arange(6)[:, None], 0.0, -30000.0)
    np.testing.assert_array_equal(host(m), exp)
    lens = dev(np.array([4, 6, 1], dtype=np.float32))
    sm = host(Ops.BuildSelfTriMask(torch.empty(3, 6, 6, device=cuda), lens, 6, 0.0, -30000.0))
    for bi, ln in enumerate([4, 6, 1]):
        q, k = np.arange(6)[:, None], np.arange(6)[None, :]
        np.testing.assert_array_equal(sm[bi], np.where((k < ln) & (q < ln) & (k <= q), 0.0, -30000.0))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL), (torch.float16, 2e-2)])
def test_addmm(cuda, oracle, dtype, tol):
    m1 = np.arange(1, 9, dtype=np.float32).reshape(2, 4)                            # GgmlOpsComparison_Tests.cs:443
    m2 = np.arange(1, 13, dtype=np.float32).reshape(4, 3)
    z = torch.zeros(2, 3, device=cuda, dtype=dtype)
    np.testing.assert_allclose(host(Ops.Addmm(None, 0.0, z, 1.0, dev(m1, dtype), dev(m2, dtype))), [[70, 80, 90], [158, 184, 210]], atol=tol * 10)
    at = dev(np.array([1, 5, 2, 6, 3, 7, 4, 8], dtype=np.float32).reshape(4, 2), dtype).t()   # :455 transposed m1
    np.testing.assert_allclose(host(Ops.Addmm(None, 0.0, z, 1.0, at, dev(m2, dtype))), [[70, 80, 90], [158, 184, 210]], atol=tol * 10)
    rng = np.random.default_rng(5)
    a = rng.standard_normal((37, 129)).astype(np.float32) * 0.3
    b = rng.standard_normal((129, 70)).astype(np.float32) * 0.3
    bias = rng.standard_normal((1, 70)).astype(np.float32)
    A, Bm, Bi = dev(a, dtype), dev(b, dtype), dev(bias, dtype)
    ref = oracle.addmm(1.0, host(Bi), 1.0, host(A), host(Bm))
    out = torch.empty(37, 70, device=cuda, dtype=dtype)
    Ops.Addmm(out, 1.0, Bi.expand(37, 70), 1.0, A, Bm)                               # Affine: bias broadcast + beta 1
    np.testing.assert_allclose(host(out), ref, atol=tol * 5)
    # batched, with a transposed second operand (Q K^T shape of attention: MultiHeadAttention.cs:209)
    q = rng.standard_normal((6, 5, 16)).astype(np.float32)
    k = rng.standard_normal((6, 9, 16)).astype(np.float32)
    Q, K = dev(q, dtype), dev(k, dtype)
    zz = torch.zeros(6, 5, 9, device=cuda, dtype=dtype)
    got = host(Ops.AddmmBatch(None, 0.0, zz, 0.25, Q, K.transpose(1, 2)))
    exp = np.stack([oracle.addmm(0.0, np.zeros((5, 9), np.float32), 0.25, host(Q)[i], host(K)[i].T.copy()) for i in range(6)])
    np.testing.assert_allclose(got, exp, atol=tol * 5)


def test_philox_matches_oracle(cuda, oracle):
    u = host(Ops.PhiloxUniform(257, seed=20261125, seq_first=5, step=3))
    exp = np.array([oracle.philox_uniform(20261125, 5 + i, 3) for i in range(257)], dtype=np.float32)
    np.testing.assert_array_equal(u, exp)


def test_errors_are_reported_not_thrown(cuda):
    a = torch.zeros(2, 3, device=cuda)
    with pytest.raises(N.TSB200Error, match="size mismatch|mismatch"):
        Ops.Addmm(None, 0.0, a, 1.0, torch.zeros(2, 4, device=cuda), torch.zeros(5, 3, device=cuda))
    with pytest.raises(N.TSB200Error, match="element type"):
        Ops.Add(None, a, a.half())
    with pytest.raises(N.TSB200Error):
        Ops.Softmax(None, torch.zeros(2, 3))  # host tensor: this backend has no CPU path
