"""The oracle's attention over an encoder output (oracle/gpt_oracle.cpp: cross_attention_block, restating
Layers/MultiHeadAttention.cs:434-527) pinned by properties that follow from the reference's formulas, and by an independent
NumPy evaluation of a one-layer model."""
import numpy as np

from oracle.cpu_oracle import OracleGPT
from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, GPTConfig, MultiHeadAttentionTypeEnums as M, NormEnums as Nm,
                                   PositionEmbeddingEnums as P, synthetic_weights)


def _cfg(**kw):
    base = dict(name="x", L=2, d=64, H=4, hd=16, F=128, V=50, norm=Nm.LayerNorm, act=A.ReLU, pe=P.RoPE, attn=M.MHA, dtype="float32",
                cross_attn=True, max_src_tokens=16)
    base.update(kw)
    return GPTConfig(**base)


def test_padding_rows_and_zero_output_projection():
    cfg = _cfg()
    w = synthetic_weights(cfg, 3, std=0.1, bias_std=0.05, max_pos=40)
    rng = np.random.default_rng(0)
    enc = rng.standard_normal((2, 7, cfg.d)).astype(np.float32)
    ids = np.array([[1], [1]], dtype=np.int32)
    o = OracleGPT(cfg, w, max_pos=40)
    o.set_encoder_output(enc, [7, 4])
    a, _ = o.step(ids)
    enc2 = enc.copy()
    enc2[1, 4:] = 99.0
    o2 = OracleGPT(cfg, w, max_pos=40)
    o2.set_encoder_output(enc2, [7, 4])
    b, _ = o2.step(ids)
    np.testing.assert_array_equal(a, b)                    # masked source rows carry exactly zero weight (exp(-30000) == 0 in fp32)
    # W0 = 0 and b0 = 0 in every cross block: the block adds nothing, the model is the plain decoder
    w0 = dict(w)
    for k in range(cfg.L):
        w0["GPTDecoder.EncAttn_%d.W0" % k] = np.zeros_like(w["GPTDecoder.EncAttn_%d.W0" % k])
        w0["GPTDecoder.EncAttn_%d.b0" % k] = np.zeros_like(w["GPTDecoder.EncAttn_%d.b0" % k])
    o3 = OracleGPT(cfg, w0, max_pos=40)
    o3.set_encoder_output(enc, [7, 4])
    c, _ = o3.step(ids)
    plain_cfg = _cfg(cross_attn=False, max_src_tokens=0)
    plain = OracleGPT(plain_cfg, {k: v for k, v in w0.items() if "EncAttn" not in k}, max_pos=40)
    d, _ = plain.step(ids)
    np.testing.assert_array_equal(c, d)
    assert np.abs(a - c).max() > 1e-3                      # and with its real weights it does change the logits


def _ln(x, g, b, eps=1e-6):
    m = x.mean(-1, keepdims=True)
    v = ((x - m) ** 2).mean(-1, keepdims=True)
    return (x - m) / np.sqrt(v + eps) * g + b


def test_one_layer_model_against_numpy():
    cfg = _cfg(L=1, pe=P.NoPE)
    w = {k: v.astype(np.float64) for k, v in synthetic_weights(cfg, 8, std=0.1, bias_std=0.05).items()}
    rng = np.random.default_rng(2)
    B, Ts, d, H, hd = 2, 5, cfg.d, cfg.H, cfg.hd
    lens = [5, 3]
    enc = rng.standard_normal((B, Ts, d))
    ids = np.array([[4], [11]], dtype=np.int32)
    o = OracleGPT(cfg, {k: v.astype(np.float32) for k, v in w.items()})
    o.set_encoder_output(enc.astype(np.float32), lens)
    got, _ = o.step(ids)
    # independent evaluation in float64: one target position, empty self-attention cache
    x = w["TgtEmbeddings"][ids[:, 0]] * np.sqrt(d)
    p = "GPTDecoder.SelfAttn_0."
    h = _ln(x, w[p + "layerNormQ.m_alpha"], w[p + "layerNormQ.m_beta"])
    qkv = h @ w[p + "QKV"] + w[p + "QKVb"]
    v_self = qkv[:, 2 * d:]                                  # a single key: softmax is 1, the context is v itself
    x = x + v_self @ w[p + "W0"] + w[p + "b0"]
    e = "GPTDecoder.EncAttn_0."
    qn = _ln(x, w[e + "layerNormQ.m_alpha"], w[e + "layerNormQ.m_beta"])
    q = (qn @ w[e + "Q"] + w[e + "Qb"]).reshape(B, H, hd)
    k = (enc @ w[e + "K"] + w[e + "Kb"]).reshape(B, Ts, H, hd)
    v = (enc @ w[e + "V"] + w[e + "Vb"]).reshape(B, Ts, H, hd)
    ctx = np.zeros((B, H, hd))
    for b in range(B):
        for hh in range(H):
            s = (k[b, :lens[b], hh] @ q[b, hh]) / np.sqrt(hd)
            a = np.exp(s - s.max())
            a /= a.sum()
            ctx[b, hh] = a @ v[b, :lens[b], hh]
    x = x + ctx.reshape(B, d) @ w[e + "W0"] + w[e + "b0"]
    f = "GPTDecoder.PosFFN_0."
    h2 = _ln(x, w[f + "layerNorm2.m_alpha"], w[f + "layerNorm2.m_beta"])
    x = x + np.maximum(h2 @ w[f + "feedForwardLayer1.m_Whd"] + w[f + "feedForwardLayer1.m_Bd"], 0) @ w[f + "feedForwardLayer2.m_Whd"] + \
        w[f + "feedForwardLayer2.m_Bd"]
    hn = _ln(x, w["GPTDecoder.layerNorm.m_alpha"], w["GPTDecoder.layerNorm.m_beta"])
    want = hn @ w["FeedForward_Decoder_0.m_Whd"] + w["FeedForward_Decoder_0.m_Bd"]
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5 * np.abs(want).max())
