"""The model file reader against files written in the reference's wire format (tests/model_file_writer.py): every
storage form (float32, float16 bit patterns, INT8 / INT4 code books), packed and element-by-element arrays, the network
shape fields, the vocabulary, and the error cases.  No GPU involved."""
import numpy as np
import pytest

from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, GPTConfig, MultiHeadAttentionTypeEnums as M, NormEnums as Nm,
                                   PositionEmbeddingEnums as P, synthetic_weights)
from seq2seqsharp_b200.model_file import ModelFileError, position_embedding, read_model
from tests.model_file_writer import write_model

CFG = GPTConfig(L=2, d=64, H=4, Hkv=2, hd=16, F=96, V=38, norm=Nm.RMSNorm, act=A.SwiGLU, pe=P.RoPE, attn=M.GQA)


def saved_weights(cfg):
    w = synthetic_weights(cfg, 5, std=0.1, bias_std=0.05)
    return {k: v for k, v in w.items() if k != "PosEmbedding"}


@pytest.mark.parametrize("packed", [True, False])
@pytest.mark.parametrize("vq", ["none", "float16", "int8", "int4"])
def test_round_trip(tmp_path, vq, packed):
    path = str(tmp_path / "m.model")
    expect = write_model(path, CFG, saved_weights(CFG), CFG.V, vq=vq, packed=packed)
    mf = read_model(path)
    assert (mf.DecoderLayerDepth, mf.HiddenDim, mf.IntermediateDim, mf.MultiHeadNum, mf.KVGroupNum) == (2, 64, 96, 4, 2)
    assert len(mf.TgtVocab) == CFG.V and mf.TgtVocab[0] == "</s>" and mf.TgtVocab[5] == "w5"
    cfg = mf.gpt_config()
    assert (cfg.L, cfg.d, cfg.H, cfg.hd, cfg.F, cfg.V, cfg.kv_heads()) == (2, 64, 4, 16, 96, 38, 2)
    assert cfg.norm == Nm.RMSNorm and cfg.act == A.SwiGLU and cfg.pe == P.RoPE and cfg.attn == M.GQA
    assert cfg.dtype == ("float16" if vq == "float16" else "float32")
    assert sorted(mf.names()) == sorted(expect)
    for name, want in expect.items():
        got = mf.get_weights(name, want_half=(vq == "float16"))
        np.testing.assert_array_equal(got.astype(np.float32), want, err_msg=name)
    shaped = mf.weights_for(cfg)
    assert shaped["GPTDecoder.SelfAttn_1.K"].shape == (64, 32) and shaped["FeedForward_Decoder_0.m_Whd"].shape == (64, 38)
    assert mf.get_weights("no.such.weight") is None


def test_float16_model_refuses_float32_request(tmp_path):
    path = str(tmp_path / "h.model")
    write_model(path, CFG, saved_weights(CFG), CFG.V, vq="float16")
    with pytest.raises(ModelFileError, match="Float16"):
        read_model(path).get_weights("TgtEmbeddings")          # Model.cs:267-270 throws InvalidCastException here


def test_mha_ape_model_and_rebuilt_position_table(tmp_path):
    cfg = GPTConfig(L=1, d=32, H=2, hd=16, F=64, V=11, norm=Nm.LayerNorm, act=A.ReLU, pe=P.APE, attn=M.MHA)
    path = str(tmp_path / "a.model")
    write_model(path, cfg, saved_weights(cfg), cfg.V)
    mf = read_model(path)
    got = mf.gpt_config()
    assert got.pe == P.APE and got.attn == M.MHA and got.kv_heads() == 2 and got.norm == Nm.LayerNorm
    w = mf.weights_for(got, max_pos=10)
    pos = w["PosEmbedding"]
    assert pos.shape == (10, 32)
    np.testing.assert_allclose(pos[0, :16], 0.0)                   # sin(0)
    np.testing.assert_allclose(pos[0, 16:], 1.0)                   # cos(0)
    np.testing.assert_allclose(pos[3, 0], np.sin(3.0), rtol=1e-6)  # the first time scale is 1
    np.testing.assert_allclose(pos[3, 15], np.sin(3.0 / 10000.0), rtol=1e-4)   # the last one 1/10000
    np.testing.assert_array_equal(position_embedding(10, 32), pos)


def test_errors(tmp_path):
    path = str(tmp_path / "e.model")
    write_model(path, CFG, saved_weights(CFG), CFG.V, decoder_type=1)
    with pytest.raises(ModelFileError, match="GPTDecoder"):
        read_model(path).gpt_config()
    write_model(path, CFG, {k: v for k, v in saved_weights(CFG).items() if not k.endswith(".W0")}, CFG.V)
    mf = read_model(path)
    with pytest.raises(ModelFileError, match="not in the model file"):
        mf.weights_for(mf.gpt_config())
    with open(path, "rb") as fh:
        data = fh.read()
    with open(path, "wb") as fh:
        fh.write(data[:len(data) // 2])
    with pytest.raises(ModelFileError):
        read_model(path)


def test_mixture_of_experts_model(tmp_path):
    """ExpertNum / ExpertsPerTokenFactor (fields 21, 22) and the tensors of MoEFeedForward (router, experts, its LayerNorm)."""
    cfg = GPTConfig(L=4, d=32, H=2, hd=16, F=64, V=38, norm=Nm.LayerNorm, act=A.SiLU, pe=P.RoPE, attn=M.MHA, expertNum=3, expertsPerTokenFactor=2)
    w = saved_weights(cfg)
    assert "GPTDecoder.MoEFFN_2.m_Whd1" in w and "GPTDecoder.PosFFN_1.feedForwardLayer1.m_Whd" in w and "GPTDecoder.PosFFN_3.feedForwardLayer1.m_Whd" not in w
    path = str(tmp_path / "moe.model")
    expect = write_model(path, cfg, w, cfg.V, vq="none")
    mf = read_model(path)
    assert (mf.ExpertNum, mf.ExpertsPerTokenFactor) == (3, 2)
    got_cfg = mf.gpt_config()
    assert (got_cfg.expertNum, got_cfg.expertsPerTokenFactor) == (3, 2) and got_cfg.is_moe_layer(2) and not got_cfg.is_moe_layer(1)
    shaped = mf.weights_for(got_cfg)
    assert shaped["GPTDecoder.MoEFFN_3.m_Whd1"].shape == (3 * 32, 128) and shaped["GPTDecoder.MoEFFN_3.m_Whd2"].shape == (3 * 128, 32)
    assert shaped["GPTDecoder.MoEFFN_2.m_Router"].shape == (32, 3) and shaped["GPTDecoder.MoEFFN_2.m_RouterBias"].shape == (1, 3)
    for name, want in expect.items():
        np.testing.assert_array_equal(mf.get_weights(name).astype(np.float32), want, err_msg=name)


def test_encoder_decoder_model_file_gives_the_decoder(tmp_path):
    """A Seq2Seq model file (DecoderType Transformer): the decoder's tensors live under "TransformerDecoder.*", the embedding
    table may be shared, and the encoder's tensors are simply not asked for."""
    cfg = GPTConfig(L=2, d=64, H=4, hd=16, F=96, V=38, norm=Nm.LayerNorm, act=A.ReLU, pe=P.APE, attn=M.MHA, cross_attn=True,
                    max_src_tokens=12)
    w = {k: v for k, v in synthetic_weights(cfg, 7, std=0.1, bias_std=0.05).items() if k != "PosEmbedding"}
    file_w = {}
    for k, v in w.items():
        if k.startswith("GPTDecoder."):
            file_w["TransformerDecoder." + k[len("GPTDecoder."):]] = v
        elif k == "TgtEmbeddings":
            file_w["SharedEmbeddings"] = v
        else:
            file_w[k] = v
    file_w["TransformerEncoder.SelfAttn_0.QKV"] = np.ones((64, 192), dtype=np.float32)      # the encoder side of the same file
    path = str(tmp_path / "s2s.model")
    expect = write_model(path, cfg, file_w, cfg.V, decoder_type=1)
    mf = read_model(path)
    with pytest.raises(ModelFileError, match="not GPTDecoder"):
        mf.gpt_config()
    got = mf.seq2seq_decoder_config(max_src_tokens=12)
    assert got.cross_attn and got.max_src_tokens == 12 and (got.L, got.d, got.H, got.hd, got.F, got.V) == (2, 64, 4, 16, 96, 38)
    assert got.attn == M.MHA and got.pe == P.APE and got.norm == Nm.LayerNorm
    shaped = mf.weights_for(got, max_pos=20)
    assert set(shaped) == set(cfg.weight_shapes(20))
    np.testing.assert_array_equal(shaped["GPTDecoder.EncAttn_1.K"].reshape(-1), expect["TransformerDecoder.EncAttn_1.K"])
    np.testing.assert_array_equal(shaped["TgtEmbeddings"].reshape(-1), expect["SharedEmbeddings"])
    assert shaped["GPTDecoder.EncAttn_0.W0"].shape == (64, 64) and shaped["PosEmbedding"].shape == (20, 64)
    # a GPT file is not an encoder-decoder file
    gpt_path = str(tmp_path / "gpt.model")
    write_model(gpt_path, CFG, saved_weights(CFG), CFG.V)
    with pytest.raises(ModelFileError, match="Transformer decoder"):
        read_model(gpt_path).seq2seq_decoder_config(8)
