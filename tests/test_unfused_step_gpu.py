"""The claim behind the unfused path - "unmodified model code runs on the op registry" - as a whole: the GPT token loop
(prompt pass and cached steps) composed ONLY from the registered op names, in the order the reference's layer code issues
them, against the oracle:

  embeddings       IndexSelect, Mul by sqrt(d)                                  (TensorUtils.cs:135-147, Decoder.cs:673,695)
  attention        LayerNorm / RMSNorm, Affine (= Copy of the expanded bias + Addmm with beta 1), views, Transpose +
                   AsContiguous, RoPE, concat-by-copy into the grown cache, MulBatch (AddmmBatch) with the scale, the
                   causal mask (BuildTriMask + Add), Softmax, MulBatch, Affine, Add  (MultiHeadAttention.cs:125-240,
                   GroupQueryAttention.cs:114-233: K / V expanded to all query heads by Expand + AsContiguous)
  feed-forward     norm, Affine, ReLU / SiLU, Affine, Add                          (PositionwiseFeedForward.cs:72-98)
  head             final norm, Affine, Softmax, Argmax                             (Decoder.cs:700-760)

torch tensors serve as device buffers with sizes and strides (views are metadata, as in TensorSharp); every arithmetic step
is an `Ops` call, i.e. one C-ABI entry point that B200BasicOps would register under that op name."""
import math

import numpy as np
import pytest
import torch

from oracle.cpu_oracle import OracleGPT
from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, GPTConfig, MultiHeadAttentionTypeEnums as M, NormEnums as Nm,
                                   PositionEmbeddingEnums as P, synthetic_weights)
from seq2seqsharp_b200.ops import Ops

pytestmark = pytest.mark.gpu

CFGS = [
    GPTConfig(name="mha_ln_relu_rope", L=2, d=128, H=4, hd=32, F=256, V=211, norm=Nm.LayerNorm, act=A.ReLU, pe=P.RoPE, attn=M.MHA, dtype="float32"),
    GPTConfig(name="gqa_rms_silu_rope", L=2, d=128, H=4, Hkv=2, hd=32, F=256, V=211, norm=Nm.RMSNorm, act=A.SiLU, pe=P.RoPE, attn=M.GQA, dtype="float32"),
]


class UnfusedGPT:
    def __init__(self, cfg, weights):
        self.c = cfg
        self.w = {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in weights.items()}
        self.cache = [None] * cfg.L          # per layer: (K [B, Hkv, T, hd], V [B, Hkv, T, hd])
        self.T = 0

    def norm(self, x, prefix):
        g = self.w[prefix + ".m_alpha"].view(-1)
        if self.c.norm == Nm.LayerNorm:
            return Ops.LayerNorm(None, x, g, self.w[prefix + ".m_beta"].view(-1), 1e-6)
        return Ops.RMSNorm(None, x, g, None, 1e-6)

    def affine(self, x, wname, bname):
        W, b = self.w[wname], self.w[bname]
        res = torch.empty(x.shape[0], W.shape[1], device="cuda")
        Ops.Copy(res, b.view(1, -1).expand(x.shape[0], W.shape[1]))          # the bias, broadcast by an expanded view
        return Ops.Addmm(res, 1.0, res, 1.0, x, W)

    def heads(self, y, B, S, n_heads):
        """[B*S, n_heads*hd] -> contiguous [B, n_heads, S, hd] (View, Transpose(1, 2), AsContiguous)."""
        return Ops.AsContiguous(y.view(B, S, n_heads, self.c.hd).transpose(1, 2))

    def concat_cache(self, old, new, T0, S):
        if old is None:
            return new
        B, Hk, _, hd = new.shape
        out = torch.empty(B, Hk, T0 + S, hd, device="cuda")
        Ops.Copy(out.narrow(2, 0, T0), old)                                    # TensorConcatenation: copies into narrowed views
        Ops.Copy(out.narrow(2, T0, S), new)
        return out

    def attention(self, k, x, B, S):
        c, T0 = self.c, self.T
        H, Hkv, hd = c.H, c.kv_heads(), c.hd
        p = "GPTDecoder.SelfAttn_%d" % k
        h = self.norm(x, p + ".layerNormQ")
        if c.attn == M.MHA:
            y = self.affine(h, p + ".QKV", p + ".QKVb").view(B, S, 3, H * hd)
            q, kk, vv = (self.heads(Ops.AsContiguous(y.select(2, i)).view(B * S, H * hd), B, S, H) for i in range(3))
        else:
            q = self.heads(self.affine(h, p + ".Q", p + ".Qb"), B, S, H)
            kk = self.heads(self.affine(h, p + ".K", p + ".Kb"), B, S, Hkv)
            vv = self.heads(self.affine(h, p + ".V", p + ".Vb"), B, S, Hkv)
        q = Ops.RoPE(None, q.view(B * H * S, hd), S, T0, c.rope_base).view(B, H, S, hd)
        kk = Ops.RoPE(None, kk.view(B * Hkv * S, hd), S, T0, c.rope_base).view(B, Hkv, S, hd)
        old = self.cache[k]
        K = self.concat_cache(old[0] if old else None, kk, T0, S)
        V = self.concat_cache(old[1] if old else None, vv, T0, S)
        self.cache[k] = (K, V)
        T1, group = T0 + S, H // Hkv
        if group > 1:   # K / V of a group serve all its query heads: Expand + AsContiguous (GroupQueryAttention.cs:156-165)
            K = Ops.AsContiguous(K.view(B * Hkv, 1, T1 * hd).expand(B * Hkv, group, T1 * hd)).view(B, H, T1, hd)
            V = Ops.AsContiguous(V.view(B * Hkv, 1, T1 * hd).expand(B * Hkv, group, T1 * hd)).view(B, H, T1, hd)
        Kt = Ops.AsContiguous(K.transpose(2, 3)).view(B * H, hd, T1)
        scores = torch.zeros(B * H, S, T1, device="cuda")
        Ops.AddmmBatch(scores, 0.0, scores, 1.0 / math.sqrt(hd), q.view(B * H, S, hd), Kt)
        if S > 1:
            mask = torch.empty(S, T1, device="cuda")
            Ops.BuildTriMask(mask, 0.0, -30000.0)
            scores = Ops.Add(None, scores, mask.view(1, S, T1).expand(B * H, S, T1))
        probs = Ops.Softmax(None, scores)
        ctx = torch.zeros(B * H, S, hd, device="cuda")
        Ops.AddmmBatch(ctx, 0.0, ctx, 1.0, probs, V.view(B * H, T1, hd))
        merged = Ops.AsContiguous(ctx.view(B, H, S, hd).transpose(1, 2)).view(B * S, H * hd)
        return Ops.Add(None, self.affine(merged, p + ".W0", p + ".b0"), x)

    def ffn(self, k, x):
        p = "GPTDecoder.PosFFN_%d" % k
        h = self.norm(x, p + ".layerNorm2")
        a = self.affine(h, p + ".feedForwardLayer1.m_Whd", p + ".feedForwardLayer1.m_Bd")
        a = Ops.Relu(None, a) if self.c.act == A.ReLU else Ops.SiLU(None, a)
        return Ops.Add(None, self.affine(a, p + ".feedForwardLayer2.m_Whd", p + ".feedForwardLayer2.m_Bd"), x)

    def step(self, ids):
        B, S = ids.shape
        idx = torch.from_numpy(ids.reshape(-1).astype(np.float32)).cuda().view(-1, 1)     # indices travel as floats in the reference
        x = Ops.IndexSelect(None, self.w["TgtEmbeddings"], idx)
        x = Ops.Mul(None, x, math.sqrt(self.c.d))
        for k in range(self.c.L):
            x = self.attention(k, x, B, S)
            x = self.ffn(k, x)
        self.T += S
        last = Ops.AsContiguous(x.view(B, S, self.c.d)[:, S - 1, :])
        hn = self.norm(last, "GPTDecoder.layerNorm")
        logits = self.affine(hn, "FeedForward_Decoder_0.m_Whd", "FeedForward_Decoder_0.m_Bd")
        probs = Ops.Softmax(None, logits)
        nxt = Ops.Argmax(None, probs, 1)
        torch.cuda.synchronize()
        return logits.cpu().numpy(), probs.cpu().numpy(), nxt.cpu().numpy().reshape(-1).astype(np.int32)


@pytest.mark.parametrize("cfg", CFGS, ids=[c.name for c in CFGS])
def test_token_loop_from_registered_ops_matches_oracle(cuda, cfg):
    w = synthetic_weights(cfg, 41, std=0.08, bias_std=0.03)
    rng = np.random.default_rng(6)
    B, S = 2, 7
    prompt = rng.integers(1, cfg.V, size=(B, S)).astype(np.int32)
    orc = OracleGPT(cfg, w, threads=2)
    dev = UnfusedGPT(cfg, w)
    ids = prompt
    for step in range(5):
        want_logits, want_probs = orc.step(ids)
        logits, probs, nxt = dev.step(ids)
        scale = float(np.abs(want_logits).max())
        assert float(np.abs(logits - want_logits).max()) <= 1e-3 * scale, step
        assert float(np.abs(probs - want_probs).max()) <= 1e-4, step
        want_next = np.argmax(want_probs, axis=1).astype(np.int32)
        top2 = np.sort(want_probs, axis=1)[:, -2:]
        for b in range(B):
            assert nxt[b] == want_next[b] or (top2[b, 1] - top2[b, 0]) < 1e-5, (step, b)
        ids = want_next[:, None]
    assert dev.T == S + 4 == orc.cache_len()
