"""NumPy twin of oracle/gpt_oracle.cpp for small cases — TEST INFRASTRUCTURE, not product code.

A second, independently written statement of the same reference semantics (float32, vectorised matmuls, so the
accumulation order differs from the C++ restatement); the CPU tests require the two to agree to ~1e-5, which
guards the C++ oracle against indexing mistakes.  Reference citations as in gpt_oracle.cpp.
"""
import math

import numpy as np

f32 = np.float32


def layernorm(x, g, b, eps):  # TensorSharp/TensorApplyCPU.cs:1360-1447
    mu = x.mean(-1, keepdims=True, dtype=f32)
    var = ((x - mu) ** 2).mean(-1, keepdims=True, dtype=f32)
    y = g * ((x - mu) / np.sqrt(f32(eps) + var))
    return (y + b if b is not None else y).astype(f32)


def rmsnorm(x, g, eps):  # TensorSharp/TensorApplyCPU.cs:1451-1496
    rms = np.sqrt((x * x).mean(-1, keepdims=True, dtype=f32) + f32(eps))
    return (g * (x / rms)).astype(f32)


def softmax(x):  # TensorSharp/TensorApplyCPU.cs:1230-1268
    e = np.exp((x - x.max(-1, keepdims=True)).astype(np.float64)).astype(f32)
    return (e / e.sum(-1, keepdims=True, dtype=f32)).astype(f32)


def rope(x, pos, base):  # x [..., S, hd], pos [S]; TensorSharp/TensorApplyCPU.cs:1148-1178
    hd = x.shape[-1]
    i = np.arange(hd // 2)
    theta = np.power(float(base), -2.0 * i / hd).astype(f32)
    ang = (theta[None, :] * pos[:, None].astype(f32)).astype(f32)
    c, s = np.cos(ang.astype(np.float64)).astype(f32), np.sin(ang.astype(np.float64)).astype(f32)
    out = np.empty_like(x)
    out[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s
    out[..., 1::2] = x[..., 1::2] * c + x[..., 0::2] * s
    return out


def act(kind, v):
    if kind == 0:
        return np.maximum(v, 0)
    if kind in (1, 4):
        return (v / (1 + np.exp(-v.astype(np.float64)))).astype(f32)
    if kind == 2:
        return np.where(v < 0, f32(0.01) * v, v)
    if kind == 5:
        from scipy.special import erf
        return (0.5 * v * (1 + erf(v.astype(np.float64) / math.sqrt(2.0)))).astype(f32)
    return v


class NpGPT:
    def __init__(self, cfg, weights):
        self.c, self.w = cfg, {k: np.asarray(v, dtype=f32) for k, v in weights.items()}
        self.reset()

    def reset(self):
        self.K = [None] * self.c.L
        self.V = [None] * self.c.L
        self.T = 0

    def _norm(self, x, prefix):
        g = self.w[prefix + ".m_alpha"].reshape(-1)
        if int(self.c.norm) == 0:
            return layernorm(x, g, self.w[prefix + ".m_beta"].reshape(-1), self.c.eps)
        return rmsnorm(x, g, self.c.eps)

    def step(self, ids, temperature=1.0, blocked=()):
        c, w = self.c, self.w
        B, S = ids.shape
        H, Hkv, hd, d = c.H, c.kv_heads(), c.hd, c.d
        T0 = self.T
        x = w["TgtEmbeddings"][ids.reshape(-1)] * f32(math.sqrt(d))        # Decoder.cs:673,695
        if int(c.pe) == 1:                                                # PositionEmbedding.cs:28-49
            pos = np.arange(S) if c.ape_decode_pos0 else np.arange(T0, T0 + S)
            x = (x.reshape(B, S, d) + w["PosEmbedding"][pos][None]).reshape(B * S, d)
        for k in range(c.L):
            a, f = "GPTDecoder.SelfAttn_%d" % k, "GPTDecoder.PosFFN_%d" % k
            h = self._norm(x, a + ".layerNormQ")
            if int(c.attn) == 0:                                          # MultiHeadAttention.cs:133-137
                qkv = (h @ w[a + ".QKV"] + w[a + ".QKVb"]).reshape(B, S, 3, H, hd)
                q, kk, vv = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
            else:                                                         # GroupQueryAttention.cs:122-124
                q = (h @ w[a + ".Q"] + w[a + ".Qb"]).reshape(B, S, H, hd)
                kk = (h @ w[a + ".K"] + w[a + ".Kb"]).reshape(B, S, Hkv, hd)
                vv = (h @ w[a + ".V"] + w[a + ".Vb"]).reshape(B, S, Hkv, hd)
            q, kk, vv = q.transpose(0, 2, 1, 3), kk.transpose(0, 2, 1, 3), vv.transpose(0, 2, 1, 3)
            if int(c.pe) == 2:
                pos = np.arange(T0, T0 + S)
                q, kk = rope(q, pos, c.rope_base), rope(kk, pos, c.rope_base)
            self.K[k] = kk if self.K[k] is None else np.concatenate([self.K[k], kk], axis=2)
            self.V[k] = vv if self.V[k] is None else np.concatenate([self.V[k], vv], axis=2)
            Kx = np.repeat(self.K[k], H // Hkv, axis=1)                   # GroupQueryAttention.cs:156-165
            Vx = np.repeat(self.V[k], H // Hkv, axis=1)
            sc = (q @ Kx.transpose(0, 1, 3, 2)) * f32(1.0 / math.sqrt(hd))
            if S > 1:                                                     # BuildTriMask 0 / -30000
                t = np.arange(T0 + S)[None, :]
                sc = sc + np.where(t <= (T0 + np.arange(S))[:, None], f32(0), f32(-30000.0))
            p = softmax(sc.astype(f32))
            o = (p @ Vx).transpose(0, 2, 1, 3).reshape(B * S, H * hd)
            x = (o @ w[a + ".W0"] + w[a + ".b0"]) + x
            h = self._norm(x, f + ".layerNorm2")
            u = act(int(c.act), (h @ w[f + ".feedForwardLayer1.m_Whd"] + w[f + ".feedForwardLayer1.m_Bd"]).astype(f32))
            if int(c.act) in (3, 4):
                u = u * (h @ w[f + ".feedForwardLayer3.m_Whd"] + w[f + ".feedForwardLayer3.m_Bd"])
            x = (u @ w[f + ".feedForwardLayer2.m_Whd"] + w[f + ".feedForwardLayer2.m_Bd"]) + x
        self.T = T0 + S
        last = x.reshape(B, S, d)[:, -1]
        hn = self._norm(last, "GPTDecoder.layerNorm")
        z = (hn @ w["FeedForward_Decoder_0.m_Whd"] + w["FeedForward_Decoder_0.m_Bd"]).astype(f32)
        if temperature != 1.0:
            z = (z / f32(temperature)).astype(f32)
        p = softmax(z)
        for b in blocked:
            p[:, b] += f32(-1.0)
        return z, p
