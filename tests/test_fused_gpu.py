"""GPU parity of the fused building blocks (decode GEMV with epilogues, residual+norm, RoPE+append, flash-decode,
prefill attention, fused softmax+argmax) against compositions of the oracle's op-level functions, through the C ABI."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from seq2seqsharp_b200 import _native as N

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    torch.cuda.synchronize()
    return t.float().cpu().numpy()


def stream():
    from seq2seqsharp_b200.ops import _stream as ops_stream
    return ops_stream()


def linear(x, W, bias, act, residual=None, dtype=torch.float32, want_f32=False):
    M, K = x.shape
    Nn = W.shape[1]
    glu = act in (N.ACT_GLU_NOACT, N.ACT_SWIGLU)
    No = Nn // 2 if glu else Nn
    y = torch.empty(M, No, device="cuda", dtype=dtype)
    y32 = torch.empty(M, No, device="cuda", dtype=torch.float32) if want_f32 else None
    wsb = N.lib().TSB200_LinearWorkspaceBytes(M, K, Nn)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    N.call("TSB200_LinearBiasAct", 0, N.F16 if dtype == torch.float16 else N.F32, y.data_ptr(),
           y32.data_ptr() if want_f32 else None, x.data_ptr(), W.data_ptr(), bias.data_ptr() if bias is not None else None,
           residual.data_ptr() if residual is not None else None, M, K, Nn, act, ws.data_ptr(), wsb, stream())
    return y32 if want_f32 else y


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 4e-3)])
@pytest.mark.parametrize("M,K,Nn", [(1, 512, 1536), (1, 4096, 6144), (3, 768, 3072), (8, 2048, 8192), (2, 11008, 4096),
                                    (1, 64, 96), (5, 100, 40), (12, 256, 512), (40, 130, 72)])
def test_linear_bias_act(cuda, oracle, dtype, tol, M, K, Nn):
    rng = np.random.default_rng(M * 131 + K + Nn)
    x = dev(rng.standard_normal((M, K)).astype(np.float32), dtype)
    W = dev((rng.standard_normal((K, Nn)) * 0.05).astype(np.float32), dtype)
    b = dev((rng.standard_normal((1, Nn)) * 0.1).astype(np.float32), dtype)
    ref = oracle.addmm(1.0, host(b), 1.0, host(x), host(W))
    scale = max(1.0, float(np.abs(ref).max()))
    np.testing.assert_allclose(host(linear(x, W, b, N.ACT_NONE, dtype=dtype)), ref, atol=tol * scale)
    np.testing.assert_allclose(host(linear(x, W, None, N.ACT_NONE, dtype=dtype)), ref - host(b), atol=tol * scale)
    for act, kind in ((N.ACT_RELU, 0), (N.ACT_SILU, 1), (N.ACT_LEAKYRELU, 2), (N.ACT_GELU, 5)):
        np.testing.assert_allclose(host(linear(x, W, b, act, dtype=dtype)), oracle.act(ref, kind), atol=tol * scale)
    # residual + fp32 output (out-proj / FFN-down epilogue)
    res = dev(rng.standard_normal((M, Nn)).astype(np.float32))
    np.testing.assert_allclose(host(linear(x, W, b, N.ACT_NONE, residual=res, dtype=dtype, want_f32=True)), ref + host(res), atol=tol * scale)
    # gated epilogue on interleaved columns (a_j, g_j)
    if Nn % 2 == 0:
        a, g = ref[:, 0::2], ref[:, 1::2]
        np.testing.assert_allclose(host(linear(x, W, b, N.ACT_GLU_NOACT, dtype=dtype)), a * g, atol=tol * scale * scale)
        np.testing.assert_allclose(host(linear(x, W, b, N.ACT_SWIGLU, dtype=dtype)), oracle.act(a, 1) * g, atol=tol * scale * scale)


def test_linear_is_bitwise_deterministic(cuda):
    rng = np.random.default_rng(0)
    x = dev(rng.standard_normal((4, 4096)).astype(np.float32), torch.float16)
    W = dev((rng.standard_normal((4096, 4096)) * 0.05).astype(np.float32), torch.float16)
    first = host(linear(x, W, None, N.ACT_NONE, dtype=torch.float16))
    for _ in range(5):
        np.testing.assert_array_equal(host(linear(x, W, None, N.ACT_NONE, dtype=torch.float16)), first)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 4e-3)])
@pytest.mark.parametrize("norm_type", [0, 1])
def test_norm_residual(cuda, oracle, dtype, tol, norm_type):
    rng = np.random.default_rng(7)
    M, d = 5, 768
    x = dev(rng.standard_normal((M, d)).astype(np.float32))
    delta = dev(rng.standard_normal((M, d)).astype(np.float32), dtype)
    g = dev(rng.standard_normal(d).astype(np.float32), dtype)
    b = dev(rng.standard_normal(d).astype(np.float32), dtype)
    x0, d0 = host(x), host(delta)
    h = torch.empty(M, d, device="cuda", dtype=dtype)
    N.call("TSB200_NormResidual", 0, N.F16 if dtype == torch.float16 else N.F32, h.data_ptr(), x.data_ptr(), delta.data_ptr(),
           g.data_ptr(), b.data_ptr() if norm_type == 0 else None, norm_type, 1e-6, M, d, stream())
    xs = x0 + d0
    np.testing.assert_allclose(host(x), xs, atol=1e-6)
    ref = oracle.layernorm(xs, host(g), host(b), 1e-6) if norm_type == 0 else oracle.rmsnorm(xs, host(g), None, 1e-6)
    np.testing.assert_allclose(host(h), ref, atol=tol * 4)


def ref_attention(oracle, q, K, V, H, Hkv, T_per_query):
    """q [B,S,H,hd]; K,V [B,Hkv,T,hd]; query s sees keys [0, T_per_query[s]).  softmax(q K^T / sqrt(hd)) V, composed from
    the oracle's addmm and softmax (MultiHeadAttention.cs:195-231)."""
    B, S, _, hd = q.shape
    out = np.zeros((B, S, H, hd), dtype=np.float32)
    scale = np.float32(1.0 / math.sqrt(hd))
    for b in range(B):
        for h in range(H):
            g = h // (H // Hkv)
            for s in range(S):
                T = T_per_query[s]
                sc = oracle.addmm(0.0, np.zeros((1, T), np.float32), float(scale), q[b, s, h][None, :], np.ascontiguousarray(K[b, g, :T].T))
                p = oracle.softmax(sc)
                out[b, s, h] = oracle.addmm(0.0, np.zeros((1, hd), np.float32), 1.0, p, np.ascontiguousarray(V[b, g, :T]))[0]
    return out


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 3e-3)])
@pytest.mark.parametrize("B,H,Hkv,hd,T", [(1, 8, 8, 64, 33), (2, 32, 8, 64, 300), (1, 32, 8, 128, 1025), (3, 4, 2, 16, 5),
                                          (2, 8, 1, 32, 700), (1, 4, 4, 64, 1),
                                          # enough (sequence, head group, split) CTAs for the cp.async-staged decode kernel:
                                          # split ranges that are not multiples of the 32-token stage, 1..5 stages per CTA
                                          (40, 32, 8, 128, 200), (64, 8, 8, 64, 77), (48, 16, 4, 128, 101), (37, 32, 32, 64, 150)])
def test_rope_append_and_flash_decode(cuda, oracle, dtype, tol, B, H, Hkv, hd, T):
    rng = np.random.default_rng(B * 1000 + T)
    dt = N.F16 if dtype == torch.float16 else N.F32
    Tmax = T + 7
    Nq = (H + 2 * Hkv) * hd
    cK = dev(rng.standard_normal((B, Hkv, Tmax, hd)).astype(np.float32), dtype)
    cV = dev(rng.standard_normal((B, Hkv, Tmax, hd)).astype(np.float32), dtype)
    qkv = dev(rng.standard_normal((B, Nq)).astype(np.float32), dtype)
    qkv0 = host(qkv)
    K0, V0 = host(cK), host(cV)
    T0 = T - 1
    N.call("TSB200_RopeAppend", 0, dt, qkv.data_ptr(), qkv.data_ptr() + H * hd * qkv.element_size(),
           qkv.data_ptr() + (H + Hkv) * hd * qkv.element_size(), Nq, Nq, cK.data_ptr(), cV.data_ptr(), B, 1, H, Hkv, hd, T0, Tmax,
           1, 500000.0, stream())
    # expected: RoPE at position T0 on q and k (reference op on rows [B*heads, S=1]), v copied
    q_ref = oracle.rope(qkv0[:, :H * hd].reshape(B * H, hd), 1, T0).reshape(B, H, hd)
    k_ref = oracle.rope(qkv0[:, H * hd:(H + Hkv) * hd].reshape(B * Hkv, hd), 1, T0).reshape(B, Hkv, hd)
    v_ref = qkv0[:, (H + Hkv) * hd:].reshape(B, Hkv, hd)
    K1, V1 = host(cK), host(cV)
    np.testing.assert_allclose(host(qkv)[:, :H * hd].reshape(B, H, hd), q_ref, atol=tol)
    np.testing.assert_allclose(K1[:, :, T0], k_ref, atol=tol)
    np.testing.assert_array_equal(V1[:, :, T0], v_ref)
    np.testing.assert_array_equal(K1[:, :, :T0], K0[:, :, :T0])      # the rest of the cache is untouched
    np.testing.assert_array_equal(K1[:, :, T0 + 1:], K0[:, :, T0 + 1:])
    # flash-decode over T cached positions
    out = torch.empty(B, H, hd, device="cuda", dtype=dtype)
    wsb = N.lib().TSB200_FlashDecodeWorkspaceBytes(B, H, hd, T)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    N.call("TSB200_FlashDecode", 0, dt, out.data_ptr(), qkv.data_ptr(), Nq, cK.data_ptr(), cV.data_ptr(), B, H, Hkv, hd, T, Tmax,
           ws.data_ptr(), wsb, stream())
    qh = host(qkv)[:, :H * hd].reshape(B, 1, H, hd)
    ref = ref_attention(oracle, qh, K1, V1, H, Hkv, [T])
    np.testing.assert_allclose(host(out).reshape(B, 1, H, hd), ref, atol=tol * 2)
    # without a workspace the kernel runs unsplit and must agree
    out2 = torch.empty_like(out)
    N.call("TSB200_FlashDecode", 0, dt, out2.data_ptr(), qkv.data_ptr(), Nq, cK.data_ptr(), cV.data_ptr(), B, H, Hkv, hd, T, Tmax,
           None, 0, stream())
    np.testing.assert_allclose(host(out2), host(out), atol=tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 3e-3)])
def test_prefill_attention_is_causal(cuda, oracle, dtype, tol):
    rng = np.random.default_rng(11)
    B, S, H, Hkv, hd = 2, 19, 8, 2, 32
    dt = N.F16 if dtype == torch.float16 else N.F32
    Tmax = 32
    Nq = (H + 2 * Hkv) * hd
    qkv = dev(rng.standard_normal((B, S, Nq)).astype(np.float32), dtype)
    cK = torch.zeros(B, Hkv, Tmax, hd, device="cuda", dtype=dtype)
    cV = torch.zeros(B, Hkv, Tmax, hd, device="cuda", dtype=dtype)
    es = qkv.element_size()
    N.call("TSB200_RopeAppend", 0, dt, qkv.data_ptr(), qkv.data_ptr() + H * hd * es, qkv.data_ptr() + (H + Hkv) * hd * es, Nq, Nq,
           cK.data_ptr(), cV.data_ptr(), B, S, H, Hkv, hd, 0, Tmax, 0, 500000.0, stream())
    out = torch.empty(B, S, H, hd, device="cuda", dtype=dtype)
    N.call("TSB200_PrefillAttention", 0, dt, out.data_ptr(), qkv.data_ptr(), Nq, cK.data_ptr(), cV.data_ptr(), B, S, H, Hkv, hd, 0,
           Tmax, stream())
    q = host(qkv)[:, :, :H * hd].reshape(B, S, H, hd)
    ref = ref_attention(oracle, q, host(cK), host(cV), H, Hkv, [s + 1 for s in range(S)])
    np.testing.assert_allclose(host(out), ref, atol=tol * 2)


def test_softmax_argmax_fused(cuda, oracle):
    rng = np.random.default_rng(5)
    B, V = 5, 32000
    z = (rng.standard_normal((B, V)) * 0.3).astype(np.float32)
    z[1, 777] = z[1].max() + 1.0
    z[2, [5, 31999]] = z[2].max() + 2.0      # exact tie in the logits: lowest index
    ids = torch.empty(B, dtype=torch.int32, device="cuda")
    probs = torch.empty(B, V, dtype=torch.float32, device="cuda")
    blocked = dev(np.array([0, 777], dtype=np.int32))
    N.call("TSB200_SoftmaxArgmax", 0, ids.data_ptr(), probs.data_ptr(), dev(z).data_ptr(), B, V, 1.0, blocked.data_ptr(), 2, stream())
    p_ref = oracle.softmax(z)
    p_ref[:, [0, 777]] += np.float32(-1.0)
    np.testing.assert_allclose(host(probs), p_ref, atol=1e-7, rtol=2e-5)
    got = host(ids).astype(np.int32)
    assert got[2] == 5 and got[1] != 777
    # the id is the first maximum of the device's own probabilities
    np.testing.assert_array_equal(got, oracle.argmax(host(probs)))
    # temperature
    N.call("TSB200_SoftmaxArgmax", 0, ids.data_ptr(), probs.data_ptr(), dev(z).data_ptr(), B, V, 0.7, None, 0, stream())
    np.testing.assert_allclose(host(probs), oracle.softmax(z / np.float32(0.7)), atol=1e-7, rtol=5e-5)


def linear_packed(x, W, bias, act, norm=None, residual=None, dtype=torch.float32, want_f32=False):
    """norm = (norm_type, gamma, beta, eps): x is then the fp32 residual stream."""
    M, K = x.shape
    Nn = W.shape[1]
    nd = N.F16 if dtype == torch.float16 else N.F32
    glu = act in (N.ACT_GLU_NOACT, N.ACT_SWIGLU)
    No = Nn // 2 if glu else Nn
    pb = N.lib().TSB200_PackedWeightBytes(nd, K, Nn)
    Wp = torch.empty(pb, dtype=torch.uint8, device="cuda")
    N.call("TSB200_PackWeight", 0, nd, Wp.data_ptr(), W.data_ptr(), N.F16 if W.dtype == torch.float16 else N.F32, K, Nn, stream())
    y = torch.empty(M, No, device="cuda", dtype=dtype)
    y32 = torch.empty(M, No, device="cuda", dtype=torch.float32) if want_f32 else None
    wsb = N.lib().TSB200_LinearPackedWorkspaceBytes(nd, M, K, Nn)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    nt, g, b, eps = norm if norm is not None else (-1, None, None, 0.0)
    N.call("TSB200_LinearPacked", 0, nd, y.data_ptr(), y32.data_ptr() if want_f32 else None,
           x.data_ptr() if norm is None else None, x.data_ptr() if norm is not None else None,
           g.data_ptr() if g is not None else None, b.data_ptr() if b is not None else None, nt, eps, Wp.data_ptr(),
           bias.data_ptr() if bias is not None else None, residual.data_ptr() if residual is not None else None, M, K, Nn, act,
           ws.data_ptr(), wsb, stream())
    return y32 if want_f32 else y


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 4e-3)])
@pytest.mark.parametrize("M,K,Nn", [(1, 512, 1536), (1, 4096, 6144), (2, 768, 3072), (4, 2048, 8192), (1, 11008, 4096),
                                    (1, 64, 96), (3, 100, 40), (1, 4096, 32000), (1, 96, 1009), (6, 256, 512), (20, 130, 72)])
def test_linear_packed_streaming_gemv(cuda, oracle, dtype, tol, M, K, Nn):
    """The TMA-fed stream-K GEMV on packed tiles (M <= 4) and the packed fallbacks (M > 4), every epilogue."""
    rng = np.random.default_rng(M * 17 + K + Nn)
    x = dev(rng.standard_normal((M, K)).astype(np.float32), dtype)
    W = dev((rng.standard_normal((K, Nn)) * 0.05).astype(np.float32), dtype)
    b = dev((rng.standard_normal((1, Nn)) * 0.1).astype(np.float32), dtype)
    ref = oracle.addmm(1.0, host(b), 1.0, host(x), host(W))
    scale = max(1.0, float(np.abs(ref).max()))
    np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_NONE, dtype=dtype)), ref, atol=tol * scale)
    np.testing.assert_allclose(host(linear_packed(x, W, None, N.ACT_RELU, dtype=dtype)), oracle.act(ref - host(b), 0), atol=tol * scale)
    np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_GELU, dtype=dtype)), oracle.act(ref, 5), atol=tol * scale)
    res = dev(rng.standard_normal((M, Nn)).astype(np.float32))
    np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_NONE, residual=res, dtype=dtype, want_f32=True)), ref + host(res), atol=tol * scale)
    if Nn % 2 == 0:
        a, g = ref[:, 0::2], ref[:, 1::2]
        np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_GLU_NOACT, dtype=dtype)), a * g, atol=tol * scale * scale)
        np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_SWIGLU, dtype=dtype)), oracle.act(a, 1) * g, atol=tol * scale * scale)
    # determinism of the stream-K reduction
    first = host(linear_packed(x, W, b, N.ACT_NONE, dtype=dtype))
    for _ in range(3):
        np.testing.assert_array_equal(host(linear_packed(x, W, b, N.ACT_NONE, dtype=dtype)), first)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 6e-3)])
@pytest.mark.parametrize("norm_type", [0, 1])
@pytest.mark.parametrize("M,K,Nn", [(1, 512, 1536), (3, 768, 2304), (1, 4096, 6144), (4, 100, 264)])
def test_linear_packed_with_fused_norm(cuda, oracle, dtype, tol, norm_type, M, K, Nn):
    rng = np.random.default_rng(K + norm_type)
    x = dev((rng.standard_normal((M, K)) * 1.7 + 0.2).astype(np.float32))
    W = dev((rng.standard_normal((K, Nn)) * 0.05).astype(np.float32), dtype)
    b = dev((rng.standard_normal((1, Nn)) * 0.1).astype(np.float32), dtype)
    g = dev((1 + 0.1 * rng.standard_normal(K)).astype(np.float32), dtype)
    be = dev((0.1 * rng.standard_normal(K)).astype(np.float32), dtype)
    h = oracle.layernorm(host(x), host(g), host(be), 1e-6) if norm_type == 0 else oracle.rmsnorm(host(x), host(g), None, 1e-6)
    if dtype == torch.float16:
        h = h.astype(np.float16).astype(np.float32)   # the normalised activations are rounded to the model dtype
    ref = oracle.addmm(1.0, host(b), 1.0, h, host(W))
    scale = max(1.0, float(np.abs(ref).max()))
    out = linear_packed(x, W, b, N.ACT_NONE, norm=(norm_type, g, be if norm_type == 0 else None, 1e-6), dtype=dtype)
    np.testing.assert_allclose(host(out), ref, atol=tol * scale)


@pytest.mark.parametrize("M,K,Nn", [(64, 64, 128), (128, 512, 256), (200, 96, 264), (17, 4096, 6144), (512, 768, 2304),
                                    (130, 1376, 512), (64, 2048, 1000), (300, 160, 96),
                                    # >= 148 tiles of 128 x 256: the persistent kernel (odd k-tile count; ragged M in one
                                    # band of 16 row tiles; a second, shorter band)
                                    (640, 160, 8000), (2000, 96, 2560), (2200, 64, 2304), (1300, 128, 4008),
                                    # 5..64 rows: the stream-K mma.sync kernel (1, 2, 4 and 8 row blocks, wide K, ragged N)
                                    (5, 4096, 4096), (12, 512, 264), (33, 1376, 512), (40, 96, 1002), (64, 11008, 4096),
                                    # 17..64 rows: the tcgen05 streaming kernel takes K >= 4096 with at least 16 M weights (whole column
                                    # tiles and halves as groups, ragged N and M); the small ones stay with the mma.sync kernels
                                    (64, 4096, 22016), (48, 128, 300), (20, 4096, 4096), (17, 256, 2304), (33, 4096, 5000)])
def test_linear_packed_tensor_core_gemm(cuda, oracle, M, K, Nn):
    """More than 4 rows on fp16 packed weights: up to 16 rows the stream-K mma.sync kernel, 17..64 rows the tcgen05 streaming
    kernel (weights as the 128-row operand; shapes it does not take fall to the mma.sync kernels), above that the tcgen05/TMEM
    GEMMs (TMA-fed, accumulator in tensor memory): every epilogue,
    ragged M (rows zero-filled by TMA), K not a multiple of the 64-wide k block, N not a multiple of the tile."""
    dtype, tol = torch.float16, 4e-3
    rng = np.random.default_rng(M + K + Nn)
    x = dev((rng.standard_normal((M, K)) * 0.5).astype(np.float32), dtype)
    W = dev((rng.standard_normal((K, Nn)) * 0.05).astype(np.float32), dtype)
    b = dev((rng.standard_normal((1, Nn)) * 0.1).astype(np.float32), dtype)
    ref = oracle.addmm(1.0, host(b), 1.0, host(x), host(W))
    scale = max(1.0, float(np.abs(ref).max()))
    np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_NONE, dtype=dtype)), ref, atol=tol * scale)
    np.testing.assert_allclose(host(linear_packed(x, W, None, N.ACT_SILU, dtype=dtype)), oracle.act(ref - host(b), 1), atol=tol * scale)
    res = dev(rng.standard_normal((M, Nn)).astype(np.float32))
    np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_NONE, residual=res, dtype=dtype, want_f32=True)), ref + host(res), atol=tol * scale)
    if Nn % 2 == 0:
        a, g = ref[:, 0::2], ref[:, 1::2]
        np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_GLU_NOACT, dtype=dtype)), a * g, atol=tol * scale * scale)
        np.testing.assert_allclose(host(linear_packed(x, W, b, N.ACT_SWIGLU, dtype=dtype)), oracle.act(a, 1) * g, atol=tol * scale * scale)
    first = host(linear_packed(x, W, b, N.ACT_NONE, dtype=dtype))
    np.testing.assert_array_equal(host(linear_packed(x, W, b, N.ACT_NONE, dtype=dtype)), first)


@pytest.mark.parametrize("M,K,N,norm", [(5, 2048, 3072, 1), (8, 2048, 512, 0), (8, 1024, 777, 1), (4, 4096, 6144, 1), (3, 4096, 1000, 0)])
def test_linear_packed_norms_up_to_eight_rows_in_the_tensor_core_kernel(cuda, oracle, M, K, N, norm, monkeypatch):
    """fp16, width 1024 / 2048 / 4096, M * width <= 16384: LayerNorm / RMSNorm of the fp32 rows inside the tensor-core
    streaming kernel (no norm launch), against the oracle's norm + affine."""
    from seq2seqsharp_b200 import _native as N_
    from seq2seqsharp_b200.ops import Ops
    import torch
    monkeypatch.setenv("TSB200_GEMV_MAXROWS", "0")      # read once per process: only effective if this test is the first caller
    rng = np.random.default_rng(M * 1000 + N)
    x32 = (rng.standard_normal((M, K)) * 1.5 + 0.3).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.03).astype(np.float16)
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    beta = (0.1 * rng.standard_normal(K)).astype(np.float16)
    bias = (0.1 * rng.standard_normal(N)).astype(np.float16)
    nd = N_.F16
    dev = lambda a: torch.from_numpy(a).cuda()
    Wd, xd, gd, bd, biasd = dev(W), dev(x32), dev(gamma), dev(beta), dev(bias)
    pb = N_.lib().TSB200_PackedWeightBytes(nd, K, N)
    Wp = torch.zeros(pb, dtype=torch.uint8, device="cuda")
    N_.call("TSB200_PackWeight", 0, nd, Wp.data_ptr(), Wd.data_ptr(), nd, K, N, None)
    y = torch.zeros(M, N, dtype=torch.float16, device="cuda")
    wsb = N_.lib().TSB200_LinearPackedWorkspaceBytes(nd, M, K, N)
    ws = torch.zeros(wsb, dtype=torch.uint8, device="cuda")
    N_.call("TSB200_LinearPacked", 0, nd, y.data_ptr(), None, None, xd.data_ptr(), gd.data_ptr(), bd.data_ptr() if norm == 0 else None, norm, 1e-6,
            Wp.data_ptr(), biasd.data_ptr(), None, M, K, N, N_.ACT_NONE, ws.data_ptr(), wsb, None)
    torch.cuda.synchronize()
    g32, b32 = gamma.astype(np.float32), beta.astype(np.float32)
    h = oracle.layernorm(x32, g32, b32, 1e-6) if norm == 0 else oracle.rmsnorm(x32, g32, None, 1e-6)
    h = h.astype(np.float16).astype(np.float32)
    want = h @ W.astype(np.float32) + bias.astype(np.float32)
    got = y.cpu().numpy().astype(np.float32)
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
