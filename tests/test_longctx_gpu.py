"""Long-context (16K+) parity: the attention kernels at the cache lengths of the long-context benchmark configuration
(batch 4, 16384-token prompts, +512 tokens: T up to 16 896), and the token loop on a 16K prompt against the CPU oracle.

Reference semantics: softmax(q K^T / sqrt(hd) + causal mask) V per head, query head h reading KV head h / (H / Hkv)
(Seq2SeqSharp/Layers/GroupQueryAttention.cs:114-233, Layers/MultiHeadAttention.cs:195-231).  The reference materialises
the [B*H, S, T] score matrix and a 4x expanded cache, so it cannot run these sizes; the expectation is computed with
NumPy in float64 per head (decode) and for a sample of query rows (prefill).  Tolerance: 6e-3 absolute on fp16 outputs
of O(1) magnitude, the bound the short-context attention tests use.
"""
import math

import numpy as np
import pytest
import torch

from seq2seqsharp_b200 import _native as N
from tests.test_fused_gpu import dev, host, stream

pytestmark = pytest.mark.gpu

TOL = 6e-3


def np_attention_rows(q, K, V, t_len):
    """q [R, hd], K/V [T, hd] float64; row r attends to keys [0, t_len[r])."""
    hd = q.shape[1]
    sc = (q @ K.T) / math.sqrt(hd)
    mask = np.arange(K.shape[0])[None, :] >= np.asarray(t_len)[:, None]
    sc = np.where(mask, -np.inf, sc)
    sc -= sc.max(axis=1, keepdims=True)
    p = np.exp(sc)
    p /= p.sum(axis=1, keepdims=True)
    return p @ V


@pytest.mark.timeout(600)
@pytest.mark.parametrize("B,H,Hkv,hd,T", [(4, 32, 8, 64, 16897), (1, 32, 8, 128, 16500), (4, 32, 8, 64, 16384 + 512)])
def test_flash_decode_at_16k(cuda, B, H, Hkv, hd, T):
    rng = np.random.default_rng(T)
    Tmax = T + 3
    Nq = (H + 2 * Hkv) * hd
    cK = dev(rng.standard_normal((B, Hkv, Tmax, hd)).astype(np.float32), torch.float16)
    cV = dev(rng.standard_normal((B, Hkv, Tmax, hd)).astype(np.float32), torch.float16)
    qkv = dev(rng.standard_normal((B, Nq)).astype(np.float32), torch.float16)
    out = torch.empty(B, H, hd, device="cuda", dtype=torch.float16)
    wsb = N.lib().TSB200_FlashDecodeWorkspaceBytes(B, H, hd, T)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    N.call("TSB200_FlashDecode", 0, N.F16, out.data_ptr(), qkv.data_ptr(), Nq, cK.data_ptr(), cV.data_ptr(), B, H, Hkv, hd, T, Tmax,
           ws.data_ptr(), wsb, stream())
    got = host(out)
    Kh, Vh, qh = host(cK).astype(np.float64), host(cV).astype(np.float64), host(qkv)[:, :H * hd].reshape(B, H, hd).astype(np.float64)
    grp = H // Hkv
    for b in range(B):
        for g in range(Hkv):
            ref = np_attention_rows(qh[b, g * grp:(g + 1) * grp], Kh[b, g, :T], Vh[b, g, :T], [T] * grp)
            np.testing.assert_allclose(got[b, g * grp:(g + 1) * grp], ref, atol=TOL)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("H,Hkv,hd,S", [(8, 2, 64, 16896), (4, 1, 128, 16400)])
def test_prefill_attention_at_16k(cuda, H, Hkv, hd, S):
    rng = np.random.default_rng(S)
    B, Tmax = 1, S + 8
    Nq = (H + 2 * Hkv) * hd
    qkv = dev(rng.standard_normal((B, S, Nq)).astype(np.float32), torch.float16)
    cK = torch.zeros(B, Hkv, Tmax, hd, device="cuda", dtype=torch.float16)
    cV = torch.zeros(B, Hkv, Tmax, hd, device="cuda", dtype=torch.float16)
    es = 2
    N.call("TSB200_RopeAppend", 0, N.F16, qkv.data_ptr(), qkv.data_ptr() + H * hd * es, qkv.data_ptr() + (H + Hkv) * hd * es, Nq, Nq,
           cK.data_ptr(), cV.data_ptr(), B, S, H, Hkv, hd, 0, Tmax, 0, 500000.0, stream())
    out = torch.empty(B, S, H, hd, device="cuda", dtype=torch.float16)
    N.call("TSB200_PrefillAttention", 0, N.F16, out.data_ptr(), qkv.data_ptr(), Nq, cK.data_ptr(), cV.data_ptr(), B, S, H, Hkv, hd, 0,
           Tmax, stream())
    got = host(out)
    assert np.isfinite(got).all()
    rows = np.unique(np.concatenate([[0, 1, 63, 64, 65, S // 2, S - 65, S - 2, S - 1], rng.integers(0, S, size=40)]))
    q = host(qkv)[0, :, :H * hd].reshape(S, H, hd).astype(np.float64)
    Kh, Vh = host(cK)[0].astype(np.float64), host(cV)[0].astype(np.float64)
    grp = H // Hkv
    for h in range(H):
        ref = np_attention_rows(q[rows, h], Kh[h // grp, :S], Vh[h // grp, :S], rows + 1)
        np.testing.assert_allclose(got[0, rows, h], ref, atol=TOL)


@pytest.mark.timeout(1200)
def test_token_loop_on_a_16k_prompt_matches_oracle(cuda, oracle):
    """Prefill of a 16 390-token prompt and greedy steps on top of it, one sequence, on a narrow one-layer model of the
    long-context configuration's architecture (RMSNorm, gated FFN, RoPE, GQA, head size 64) — the widest the oracle's
    materialised score matrix allows.  Positions, the RoPE table, split counts and the cache append run at 16K."""
    from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, DecodingOptions, GPTConfig, MultiHeadAttentionTypeEnums as M,
                                       NormEnums as Nm, PositionEmbeddingEnums as P, synthetic_weights)
    from seq2seqsharp_b200.synthetic import prompt_ids
    from tests.test_gpt_gpu import compare_run, run_pair
    cfg = GPTConfig(name="c4_arch_narrow", L=1, d=128, H=2, Hkv=1, hd=64, F=256, V=997, norm=Nm.RMSNorm, act=A.SwiGLU, pe=P.RoPE,
                    attn=M.GQA, dtype="float16")
    w = synthetic_weights(cfg, 3, std=0.05)
    S, n_new = 16390, 6
    prompt = prompt_ids(5, 1, S, cfg.V)
    opts = DecodingOptions(MaxTgtSentLength=S + n_new, BlockedTokens=[0])
    o_ids, steps, d_ids, d_logits = run_pair(oracle, cfg, w, prompt, opts, 0, threads=oracle.max_threads())
    print("ties:", compare_run(oracle, cfg, o_ids, steps, d_ids, d_logits, opts, prompt))
