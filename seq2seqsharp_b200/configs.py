"""The five benchmark configurations (shapes from the project's baseline description), expressed with the
reference's own switches.  Where the baseline prose and the reference disagree the reference wins by default
(RoPE base 500000, eps 1e-6, "SwiGLU" without SiLU, fixed sinusoid APE added at row 0 in cached decode); the
prose variants are reachable through GPTConfig fields."""
from .gpt import (ActivateFuncEnums as A, GPTConfig, MultiHeadAttentionTypeEnums as M, NormEnums as Nm,
                  PositionEmbeddingEnums as P)

C1_TINY = GPTConfig(name="c1_tiny_fp32", L=6, d=512, H=8, hd=64, F=2048, V=32000, norm=Nm.LayerNorm, act=A.ReLU,
                    pe=P.RoPE, attn=M.MHA, dtype="float32")
C2_GPT2S = GPTConfig(name="c2_gpt2small_fp16", L=12, d=768, H=12, hd=64, F=3072, V=50257, norm=Nm.LayerNorm,
                     act=A.GELU, pe=P.APE, attn=M.MHA, dtype="float16")
C3_LLAMA1B = GPTConfig(name="c3_llama1b_fp16", L=16, d=2048, H=32, Hkv=8, hd=64, F=8192, V=32000, norm=Nm.RMSNorm,
                       act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16")
C4_LONGCTX = GPTConfig(name="c4_llama1b_longctx_fp16", L=16, d=2048, H=32, Hkv=8, hd=64, F=8192, V=32000,
                       norm=Nm.RMSNorm, act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16")
C5_LLAMA7B = GPTConfig(name="c5_llama7b_fp16", L=32, d=4096, H=32, Hkv=8, hd=128, F=11008, V=32000, norm=Nm.RMSNorm,
                       act=A.SwiGLU, pe=P.RoPE, attn=M.GQA, dtype="float16")

CONFIGS = {c.name: c for c in (C1_TINY, C2_GPT2S, C3_LLAMA1B, C4_LONGCTX, C5_LLAMA7B)}
SEED = 20261125


def shrink(cfg: GPTConfig, L=2, d=None, F=None, V=None, H=None, Hkv=None):
    """A small model with the same architecture switches (for parity tests the CPU oracle finishes in seconds)."""
    import dataclasses
    H = H or cfg.H
    return dataclasses.replace(cfg, name=cfg.name + "_small", L=L, d=d or H * cfg.hd, F=F or cfg.F, V=V or cfg.V, H=H,
                               Hkv=Hkv if Hkv is not None else cfg.Hkv)
