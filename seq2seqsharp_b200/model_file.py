"""Reader of the reference's model file, straight into the B200 engine.

Seq2SeqSharp saves a model as ONE protobuf-net message, `Model_4_ProtoBufSerializer`
(Seq2SeqSharp/Models/Model_4_ProtoBufSerializer.cs:233-323): the network shape (field numbers 2-11, 23, 28-31), the
vocabularies (12-14) and the weights by name in four dictionaries:

    1  Name2Weights      string -> float[]    full-precision weights
    27 Name2WeightsHalf  string -> ushort[]   fp16 bit patterns              (VQType FLOAT16)
    25 Name2WeightsVQ    string -> byte[]     code-book indices              (VQType INT8: one per weight;
    26 Name2CodeBook     string -> double[]   256 / 16 code-book values       INT4: two per byte, low nibble first)

`Model.GetWeights` (Seq2SeqSharp/Models/Model.cs:258-312) is the decoding rule restated in `ModelFile.get_weights`.
protobuf-net writes a dictionary as a repeated sub-message {1: key, 2: value} on the member's field number and an array
of scalars as a repeated field, packed or not depending on version and options, so both encodings are accepted.  The
fixed sinusoid position table is not stored in the file (`isStaticWeights`, Seq2SeqSharp/Utils/PositionEmbedding.cs:
51-72); `position_embedding` rebuilds it.

Only the Python standard library and NumPy are used: no protobuf runtime, no .NET.
"""
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from .gpt import (ActivateFuncEnums, GPTConfig, MultiHeadAttentionTypeEnums, NormEnums, PositionEmbeddingEnums)

# field numbers of Model_4_ProtoBufSerializer
F_WEIGHTS, F_DEC_EMB, F_ENC_EMB, F_DEC_DEPTH, F_ENC_DEPTH, F_DEC_TYPE, F_ENC_TYPE, F_HIDDEN, F_INTER = 1, 2, 3, 4, 5, 6, 7, 8, 9
F_SEG, F_HEADS, F_SRC_VOCAB, F_TGT_VOCAB, F_CLS_VOCABS = 10, 11, 12, 13, 14
F_EXPERTS, F_ACT, F_VQTYPE, F_VQ, F_CODEBOOK, F_HALF, F_PE, F_NORM, F_MHA_TYPE, F_KV_GROUPS = 21, 23, 24, 25, 26, 27, 28, 29, 30, 31
F_EXPERTS_PER_TOKEN = 22
VQ_NONE, VQ_INT4, VQ_INT8, VQ_FLOAT16 = 0, 16, 256, 65536          # Seq2SeqSharp/Utils/ModeEnums.cs:41-47
DECODER_GPT = 2                                                    # DecoderTypeEnums.GPTDecoder
DECODER_TRANSFORMER = 1                                            # DecoderTypeEnums.Transformer (Utils/ModeEnums.cs:33-39)


class ModelFileError(ValueError):
    pass


def _varint(buf, pos):
    result = shift = 0
    while True:
        if pos >= len(buf):
            raise ModelFileError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise ModelFileError("varint too long")


def _fields(buf):
    """Yields (field number, wire type, value) of one message; value is an int (varint / fixed) or a memoryview."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        fno, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _varint(buf, pos)
        elif wt == 1:
            v, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            if pos + ln > n:
                raise ModelFileError("field %d: length %d exceeds the message" % (fno, ln))
            v, pos = buf[pos:pos + ln], pos + ln
        elif wt == 5:
            v, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ModelFileError("unsupported wire type %d (field %d)" % (wt, fno))
        yield fno, wt, v


def _signed(v):
    return v - (1 << 64) if v >= 1 << 63 else v


def _pair(buf, value_kind):
    """One dictionary entry {1: key, 2: value}.  value_kind: 'f32' | 'f64' | 'u16' | 'bytes' | 'int' | 'str'."""
    key, packed, singles = None, [], []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            key = bytes(v).decode("utf-8") if wt == 2 else _signed(v)
        elif fno == 2:
            if value_kind == "bytes":
                packed.append(bytes(v))
            elif value_kind == "str":
                singles.append(bytes(v).decode("utf-8"))
            elif value_kind == "int":
                singles.append(_signed(v))
            elif wt == 2:
                packed.append(bytes(v))          # packed repeated scalars
            elif value_kind == "u16":
                singles.append(v)                # one varint per element
            else:
                singles.append(bytes(v))         # one fixed32 / fixed64 per element
    if value_kind == "bytes":
        val = np.frombuffer(b"".join(packed), dtype=np.uint8)
    elif value_kind in ("str", "int"):
        val = singles[0] if singles else ("" if value_kind == "str" else 0)
    elif value_kind == "u16":
        if packed:
            raw, out, pos = b"".join(packed), [], 0
            while pos < len(raw):
                x, pos = _varint(raw, pos)
                out.append(x)
            val = np.asarray(out, dtype=np.uint16)
        else:
            val = np.asarray(singles, dtype=np.uint16)
    else:
        dt = np.dtype("<f4") if value_kind == "f32" else np.dtype("<f8")
        val = np.frombuffer(b"".join(packed) if packed else b"".join(singles), dtype=dt)
    return key, val


@dataclass
class ModelFile:
    DecoderEmbeddingDim: int = 0
    EncoderEmbeddingDim: int = 0
    DecoderLayerDepth: int = 0
    EncoderLayerDepth: int = 0
    DecoderType: int = 0
    EncoderType: int = 0
    HiddenDim: int = 0
    IntermediateDim: int = 0
    MultiHeadNum: int = 0
    ExpertNum: int = 0
    ExpertsPerTokenFactor: int = 0
    ActivateFunc: int = 0
    VQType: int = 0
    PEType: int = 0
    NormType: int = 0
    MultiHeadAttentionType: int = 0
    KVGroupNum: int = 0
    Name2Weights: Dict[str, np.ndarray] = field(default_factory=dict)
    Name2WeightsHalf: Dict[str, np.ndarray] = field(default_factory=dict)
    Name2WeightsVQ: Dict[str, np.ndarray] = field(default_factory=dict)
    Name2CodeBook: Dict[str, np.ndarray] = field(default_factory=dict)
    TgtVocab: Optional[List[str]] = None
    SrcVocab: Optional[List[str]] = None

    def names(self):
        return sorted(set(self.Name2Weights) | set(self.Name2WeightsHalf) | set(self.Name2WeightsVQ))

    def get_weights(self, name: str, want_half: bool = False) -> Optional[np.ndarray]:
        """Model.GetWeights / GetWeightsHalfType: float32 (or float16 with want_half) values of a weight, or None.
        As in the reference, a model saved as FLOAT16 refuses a float32 request."""
        if name in self.Name2Weights:
            w = self.Name2Weights[name]
            return w.astype(np.float16) if want_half else w.astype(np.float32)
        if name in self.Name2WeightsHalf:
            if not want_half:
                raise ModelFileError("the model is saved as Float16: load it with a float16 engine (Model.cs:267-270)")
            return self.Name2WeightsHalf[name].view(np.float16)
        if name in self.Name2WeightsVQ:
            idx, book = self.Name2WeightsVQ[name], self.Name2CodeBook[name]
            if self.VQType == VQ_INT8:
                w = book[idx]
            elif self.VQType == VQ_INT4:
                w = np.empty(idx.size * 2, dtype=np.float64)
                w[0::2] = book[idx & 0x0F]         # low nibble first (Model.cs:241-245, 296-302)
                w[1::2] = book[idx >> 4]
            else:
                raise ModelFileError("vector-quantised weights in a model whose VQType is %d" % self.VQType)
            return w.astype(np.float16 if want_half else np.float32)
        return None

    def gpt_config(self, dtype: Optional[str] = None) -> GPTConfig:
        """The GPTDecoder this file describes, in the engine's terms (GPT.cs:112-134 builds the network from these fields)."""
        if self.DecoderType != DECODER_GPT:
            raise ModelFileError("DecoderType %d is not GPTDecoder: only the GPT decode path runs on this backend" % self.DecoderType)
        if self.MultiHeadNum <= 0 or self.HiddenDim % self.MultiHeadNum:
            raise ModelFileError("HiddenDim %d is not divisible by MultiHeadNum %d" % (self.HiddenDim, self.MultiHeadNum))
        if self.TgtVocab is None:
            raise ModelFileError("the file holds no target vocabulary, so the LM head width is unknown")
        pe = {0: PositionEmbeddingEnums.APE, 1: PositionEmbeddingEnums.NoPE, 2: PositionEmbeddingEnums.RoPE}[self.PEType]   # Utils/PositionEmbedding.cs:18-23
        gqa = self.MultiHeadAttentionType == 1
        if dtype is None:
            dtype = "float16" if self.VQType == VQ_FLOAT16 else "float32"
        return GPTConfig(L=self.DecoderLayerDepth, d=self.HiddenDim, H=self.MultiHeadNum, hd=self.HiddenDim // self.MultiHeadNum,
                         F=self.IntermediateDim, V=len(self.TgtVocab), Hkv=self.KVGroupNum if gqa else 0,
                         norm=NormEnums(self.NormType), act=ActivateFuncEnums(self.ActivateFunc), pe=pe,
                         attn=MultiHeadAttentionTypeEnums.GQA if gqa else MultiHeadAttentionTypeEnums.MHA, dtype=dtype, name="model_file",
                         expertNum=max(1, self.ExpertNum), expertsPerTokenFactor=max(1, self.ExpertsPerTokenFactor))

    def seq2seq_decoder_config(self, max_src_tokens: int, dtype: Optional[str] = None) -> GPTConfig:
        """The TransformerDecoder of an encoder-decoder model file (Applications/Decoder.cs:45-52 builds it from these fields):
        MultiHeadAttention self-attention, attention over the encoder output, feed-forward.  The encoder's tensors of the same
        file are not used by this backend: the encoder output is an input of the decoder path."""
        if self.DecoderType != DECODER_TRANSFORMER:
            raise ModelFileError("DecoderType %d is not the Transformer decoder of an encoder-decoder model" % self.DecoderType)
        if self.MultiHeadNum <= 0 or self.HiddenDim % self.MultiHeadNum:
            raise ModelFileError("HiddenDim %d is not divisible by MultiHeadNum %d" % (self.HiddenDim, self.MultiHeadNum))
        if self.TgtVocab is None:
            raise ModelFileError("the file holds no target vocabulary, so the LM head width is unknown")
        pe = {0: PositionEmbeddingEnums.APE, 1: PositionEmbeddingEnums.NoPE, 2: PositionEmbeddingEnums.RoPE}[self.PEType]
        if dtype is None:
            dtype = "float16" if self.VQType == VQ_FLOAT16 else "float32"
        return GPTConfig(L=self.DecoderLayerDepth, d=self.HiddenDim, H=self.MultiHeadNum, hd=self.HiddenDim // self.MultiHeadNum,
                         F=self.IntermediateDim, V=len(self.TgtVocab), norm=NormEnums(self.NormType), act=ActivateFuncEnums(self.ActivateFunc),
                         pe=pe, attn=MultiHeadAttentionTypeEnums.MHA, dtype=dtype, name="model_file_seq2seq_decoder", cross_attn=True,
                         max_src_tokens=int(max_src_tokens))

    def _file_name(self, cfg: GPTConfig, name: str) -> str:
        """The key under which the file stores what the engine calls `name`: an encoder-decoder model names its decoder
        "TransformerDecoder" and may keep one embedding table for both sides ("SharedEmbeddings")."""
        if not cfg.cross_attn:
            return name
        if name.startswith("GPTDecoder."):
            return "TransformerDecoder." + name[len("GPTDecoder."):]
        if name == "TgtEmbeddings" and name not in self.names() and "SharedEmbeddings" in self.names():
            return "SharedEmbeddings"
        return name

    def weights_for(self, cfg: GPTConfig, max_pos: int = 0) -> Dict[str, np.ndarray]:
        """Every tensor the engine asks for, shaped [rows, cols], in the file's own precision (float16 arrays for a
        FLOAT16 file, float32 otherwise).  Missing tensors are an error; PosEmbedding is rebuilt."""
        half = bool(self.Name2WeightsHalf)
        out = {}
        for name, shape in cfg.weight_shapes(max_pos).items():
            if name == "PosEmbedding":
                out[name] = position_embedding(shape[0], shape[1])
                continue
            w = self.get_weights(self._file_name(cfg, name), want_half=half)
            if w is None:
                raise ModelFileError("weight '%s' is not in the model file" % name)
            if w.size != shape[0] * shape[1]:
                raise ModelFileError("weight '%s' has %d values, the network needs %d x %d" % (name, w.size, shape[0], shape[1]))
            out[name] = np.ascontiguousarray(w).reshape(shape)
        return out


def position_embedding(rows: int, cols: int) -> np.ndarray:
    """PositionEmbedding.BuildPositionWeightTensor (Utils/PositionEmbedding.cs:51-72): sin in the first half of the columns,
    cos in the second, float32 arithmetic as in the reference."""
    n = cols // 2
    inc = np.float32(math.log(np.float32(10000.0)) / (np.float32(n) - np.float32(1.0)))
    out = np.zeros((rows, cols), dtype=np.float32)
    i = np.arange(n, dtype=np.float64)
    scale = np.exp(i * -np.float64(inc))
    for p in range(rows):
        v = (p * scale).astype(np.float32).astype(np.float64)
        out[p, :n] = np.sin(v)
        out[p, n:2 * n] = np.cos(v)
    return out


def _vocab(buf) -> List[str]:
    """Vocab_4_ProtoBufSerializer (Model_4_ProtoBufSerializer.cs:19-23): 1 word -> index, 2 index -> word, 3 ignore case."""
    by_index, by_word = {}, {}
    for fno, wt, v in _fields(buf):
        if fno == 2 and wt == 2:
            k, w = _pair(v, "str")
            by_index[int(k)] = w
        elif fno == 1 and wt == 2:
            w, k = _pair(v, "int")
            by_word[w] = int(k)
    if not by_index:
        by_index = {i: w for w, i in by_word.items()}
    return [by_index.get(i, "") for i in range(max(by_index) + 1)] if by_index else []


def parse_model(data) -> ModelFile:
    buf = memoryview(data)
    m = ModelFile()
    scalars = {F_DEC_EMB: "DecoderEmbeddingDim", F_ENC_EMB: "EncoderEmbeddingDim", F_DEC_DEPTH: "DecoderLayerDepth",
               F_ENC_DEPTH: "EncoderLayerDepth", F_DEC_TYPE: "DecoderType", F_ENC_TYPE: "EncoderType", F_HIDDEN: "HiddenDim",
               F_INTER: "IntermediateDim", F_HEADS: "MultiHeadNum", F_EXPERTS: "ExpertNum", F_EXPERTS_PER_TOKEN: "ExpertsPerTokenFactor", F_ACT: "ActivateFunc", F_VQTYPE: "VQType",
               F_PE: "PEType", F_NORM: "NormType", F_MHA_TYPE: "MultiHeadAttentionType", F_KV_GROUPS: "KVGroupNum"}
    for fno, wt, v in _fields(buf):
        if fno in scalars and wt == 0:
            setattr(m, scalars[fno], int(_signed(v)))
        elif wt != 2:
            continue
        elif fno == F_WEIGHTS:
            k, w = _pair(v, "f32")
            m.Name2Weights[k] = w
        elif fno == F_HALF:
            k, w = _pair(v, "u16")
            m.Name2WeightsHalf[k] = w
        elif fno == F_VQ:
            k, w = _pair(v, "bytes")
            m.Name2WeightsVQ[k] = w
        elif fno == F_CODEBOOK:
            k, w = _pair(v, "f64")
            m.Name2CodeBook[k] = w
        elif fno == F_TGT_VOCAB:
            m.TgtVocab = _vocab(v)
        elif fno == F_SRC_VOCAB:
            m.SrcVocab = _vocab(v)
    return m


def read_model(path: str) -> ModelFile:
    with open(path, "rb") as fh:
        return parse_model(fh.read())


def load_seq2seq_decoder(path: str, max_src_tokens: int, device_id: int = 0, max_batch: int = 1, max_tokens: int = 512,
                         dtype: Optional[str] = None):
    """Encoder-decoder model file -> an engine holding its decoder (self-attention, attention over the encoder output,
    feed-forward, LM head); the encoder output arrives through `GPT.SetEncoderOutput`.  Returns (GPT, ModelFile)."""
    from .gpt import GPT
    mf = read_model(path)
    cfg = mf.seq2seq_decoder_config(max_src_tokens, dtype)
    gpt = GPT(cfg, device_id=device_id, max_batch=max_batch, max_tokens=max_tokens)
    gpt.LoadWeights(mf.weights_for(cfg, gpt.pos_embedding_rows if cfg.pe == PositionEmbeddingEnums.APE else 0))
    return gpt, mf


def load_gpt(path: str, device_id: int = 0, max_batch: int = 1, max_tokens: int = 512, dtype: Optional[str] = None):
    """Model file -> a ready engine: what `GPT(options)` + `LoadModel` do in the reference (Applications/GPT.cs:48-110),
    with the weights handed to TSB200_GptSetWeight by their reference names.  Returns (GPT, ModelFile)."""
    from .gpt import GPT
    mf = read_model(path)
    cfg = mf.gpt_config(dtype)
    gpt = GPT(cfg, device_id=device_id, max_batch=max_batch, max_tokens=max_tokens)
    gpt.LoadWeights(mf.weights_for(cfg, gpt.pos_embedding_rows if cfg.pe == PositionEmbeddingEnums.APE else 0))
    return gpt, mf
