"""Writer of the reference's model file format (a protobuf-net `Model_4_ProtoBufSerializer` message,
Seq2SeqSharp/Models/Model_4_ProtoBufSerializer.cs:233-323) — test support for the reader in
seq2seqsharp_b200/model_file.py.  It produces small files on the fly; nothing of a real model is stored.

`packed` chooses how arrays of scalars are written: True = one length-delimited blob per array (protobuf "packed"
encoding), False = one tagged element after another (what protobuf-net emits for arrays without IsPacked)."""
import struct

import numpy as np


def _varint(v):
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(fno, wt):
    return _varint((fno << 3) | wt)


def _ld(fno, payload):
    return _key(fno, 2) + _varint(len(payload)) + payload


def _scalars(fno, arr, kind, packed):
    if kind == "f32":
        raw = [struct.pack("<f", float(x)) for x in arr]
        return _ld(fno, b"".join(raw)) if packed else b"".join(_key(fno, 5) + r for r in raw)
    if kind == "f64":
        raw = [struct.pack("<d", float(x)) for x in arr]
        return _ld(fno, b"".join(raw)) if packed else b"".join(_key(fno, 1) + r for r in raw)
    raw = [_varint(int(x)) for x in arr]   # u16 as varints
    return _ld(fno, b"".join(raw)) if packed else b"".join(_key(fno, 0) + r for r in raw)


def _entry(fno, key, value_bytes):
    return _ld(fno, _ld(1, key.encode("utf-8")) + value_bytes)


def _vocab(words):
    body = b""
    for i, w in enumerate(words):
        body += _ld(1, _ld(1, w.encode("utf-8")) + _key(2, 0) + _varint(i))
        body += _ld(2, _key(1, 0) + _varint(i) + _ld(2, w.encode("utf-8")))
    return body + _key(3, 0) + _varint(0)


def quantize(w, levels):
    """A simple code book (equally spaced quantiles) and the index of the nearest entry — stands in for the reference's
    VectorQuantization.BuildCodebook; the READER only needs indices + code book."""
    flat = np.asarray(w, dtype=np.float64).reshape(-1)
    book = np.quantile(flat, (np.arange(levels) + 0.5) / levels)
    idx = np.abs(flat[:, None] - book[None, :]).argmin(axis=1).astype(np.uint8)
    return book, idx


def write_model(path, cfg, weights, vocab_size, vq="none", packed=True, decoder_type=2):
    """weights: name -> float32 array (any shape); vq: 'none' | 'float16' | 'int8' | 'int4'.
    Returns the weights as the READER must reproduce them (float32; after quantisation / rounding)."""
    pe = {1: 0, 0: 1, 2: 2}[int(cfg.pe)]       # engine numbering NoPE 0 / APE 1 / RoPE 2 -> file numbering APE 0 / NoPE 1 / RoPE 2
    vqtype = {"none": 0, "float16": 65536, "int8": 256, "int4": 16}[vq]
    out = bytearray()
    expect = {}
    for name, w in weights.items():
        flat = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
        if vq == "none":
            out += _entry(1, name, _scalars(2, flat, "f32", packed))
            expect[name] = flat.copy()
        elif vq == "float16":
            h = flat.astype(np.float16)
            out += _entry(27, name, _scalars(2, h.view(np.uint16), "u16", packed))
            expect[name] = h.astype(np.float32)
        else:
            levels = 256 if vq == "int8" else 16
            book, idx = quantize(flat, levels)
            if vq == "int4":
                assert flat.size % 2 == 0
                by = (idx[1::2].astype(np.uint8) * 16 + idx[0::2]).astype(np.uint8)   # high * 16 + low (Model.cs:241-245)
            else:
                by = idx
            out += _entry(25, name, _ld(2, by.tobytes()))
            out += _entry(26, name, _scalars(2, book, "f64", packed))
            expect[name] = book[idx].astype(np.float32)
    for fno, v in ((2, cfg.d), (3, cfg.d), (4, cfg.L), (5, 0), (6, decoder_type), (8, cfg.d), (9, cfg.F), (11, cfg.H),
                   (21, cfg.expertNum if cfg.expertNum > 1 else 0), (22, cfg.expertsPerTokenFactor if cfg.expertNum > 1 else 0), (23, int(cfg.act)),
                   (24, vqtype), (28, pe), (29, int(cfg.norm)), (30, int(cfg.attn)), (31, cfg.kv_heads() if int(cfg.attn) == 1 else 0)):
        if v:   # protobuf-net leaves default (zero) values out
            out += _key(fno, 0) + _varint(v)
    out += _ld(13, _vocab(["</s>"] + ["w%d" % i for i in range(1, vocab_size)]))
    with open(path, "wb") as fh:
        fh.write(bytes(out))
    return expect
