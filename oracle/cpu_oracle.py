"""ctypes wrapper of oracle/liboracle.so — TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
Build: `make -C oracle` (done by __graft_entry__.build()).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")


class OrcConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("L", "d", "H", "Hkv", "hd", "F", "V", "norm_type", "act", "pe_type",
                                          "attn_type")] + [("eps", C.c_float), ("rope_base", C.c_float)] + \
               [(n, C.c_int32) for n in ("ape_decode_pos0", "max_pos", "faithful_cache", "threads", "n_experts", "experts_per_token",
                                         "cross_attn")]


_lib = None


def build():
    subprocess.run(["make", "-C", _HERE, "-s"], check=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_HERE, "gpt_oracle.cpp")):
            build()
        L = C.CDLL(_LIB)
        fp, ip, vp = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_void_p
        L.orc_create.restype = vp
        L.orc_create.argtypes = [C.POINTER(OrcConfig)]
        L.orc_destroy.argtypes = [vp]
        L.orc_set_weight.restype = C.c_int
        L.orc_set_weight.argtypes = [vp, C.c_char_p, fp, C.c_int, C.c_int]
        L.orc_reset.argtypes = [vp]
        L.orc_cache_len.restype = C.c_int
        L.orc_cache_len.argtypes = [vp]
        L.orc_set_encoder_output.restype = C.c_int
        L.orc_set_encoder_output.argtypes = [vp, fp, ip, C.c_int, C.c_int]
        L.orc_step.restype = C.c_int
        L.orc_step.argtypes = [vp, ip, C.c_int, C.c_int, C.c_float, ip, C.c_int, fp, fp, fp]
        L.orc_layernorm.argtypes = [fp, fp, fp, fp, C.c_float, C.c_int, C.c_int]
        L.orc_rmsnorm.argtypes = [fp, fp, fp, fp, C.c_float, C.c_int, C.c_int]
        L.orc_softmax.argtypes = [fp, fp, C.c_int, C.c_int]
        L.orc_rope.argtypes = [fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double]
        L.orc_argmax.argtypes = [ip, fp, C.c_int, C.c_int]
        L.orc_addmm.argtypes = [fp, C.c_float, fp, C.c_float, fp, fp, C.c_int, C.c_int, C.c_int]
        L.orc_act.argtypes = [fp, fp, C.c_long, C.c_int]
        L.orc_indexselect.argtypes = [fp, fp, fp, C.c_int, C.c_int]
        L.orc_topp.argtypes = [ip, fp, C.c_int, C.c_int, C.c_float, C.c_float, ip, ip, C.c_int, fp, ip, fp]
        L.orc_philox4x32_10.argtypes = [C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        L.orc_philox_uniform.restype = C.c_float
        L.orc_philox_uniform.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32]
        L.orc_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _c32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def layernorm(x, gamma, beta, eps):
    x = _c32(x); out = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_layernorm(_f(out), _f(x), _f(_c32(gamma)), _f(_c32(beta)) if beta is not None else None, eps, x.size // cols, cols)
    return out


def rmsnorm(x, gamma, beta, eps):
    x = _c32(x); out = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_rmsnorm(_f(out), _f(x), _f(_c32(gamma)), _f(_c32(beta)) if beta is not None else None, eps, x.size // cols, cols)
    return out


def softmax(x):
    x = _c32(x); out = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_softmax(_f(out), _f(x), x.size // cols, cols)
    return out


def rope(x, seq_len, row_offset, base=500000.0):
    x = _c32(x); out = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_rope(_f(out), _f(x), x.size // cols, cols, seq_len, row_offset, base)
    return out


def topk(x, k):
    """TensorApplyCPU.TopK (TensorSharp/TensorApplyCPU.cs:1121-1146): values and indices of the k largest entries of every
    row, descending; a value equal to the current k-th replaces it."""
    x = _c32(x)
    rows, cols = x.shape
    val = np.empty((rows, k), dtype=np.float32)
    idx = np.empty((rows, k), dtype=np.int32)
    L = lib()
    L.orc_topk.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_float), C.c_int, C.c_int, C.c_int]
    L.orc_topk(_f(val), _i(idx), _f(x), rows, cols, k)
    return val, idx


def argmax(p):
    p = _c32(p)
    cols = p.shape[-1]
    out = np.empty(p.size // cols, dtype=np.int32)
    lib().orc_argmax(_i(out), _f(p), p.size // cols, cols)
    return out


def addmm(beta, src, alpha, a, b):
    a, b = _c32(a), _c32(b)
    M, K = a.shape
    N = b.shape[1]
    src = _c32(np.broadcast_to(src, (M, N)))
    out = np.empty((M, N), dtype=np.float32)
    lib().orc_addmm(_f(out), beta, _f(src), alpha, _f(a), _f(b), M, K, N)
    return out


def act(x, kind):
    x = _c32(x); out = np.empty_like(x)
    lib().orc_act(_f(out), _f(x), x.size, kind)
    return out


def indexselect(src, idx, out=None):
    src = _c32(src); idx = _c32(idx).reshape(-1)
    if out is None:
        out = np.zeros((idx.size, src.shape[1]), dtype=np.float32)
    lib().orc_indexselect(_f(out), _f(src), _f(idx), idx.size, src.shape[1])
    return out


def topp(probs, topP, repeat_penalty, seqs, u, return_details=False):
    probs = _c32(probs)
    B, V = probs.shape
    u = _c32(u)
    out = np.empty(B, dtype=np.int32)
    ncand = np.empty(B, dtype=np.int32)
    acc = np.empty(B, dtype=np.float32)
    if seqs is not None:
        stride = max(1, max(len(s) for s in seqs))
        h = np.zeros((B, stride), dtype=np.int32)
        for i, s in enumerate(seqs):
            h[i, :len(s)] = s
        lens = np.array([len(s) for s in seqs], dtype=np.int32)
        lib().orc_topp(_i(out), _f(probs), B, V, topP, repeat_penalty, _i(h), _i(lens), stride, _f(u), _i(ncand), _f(acc))
    else:
        lib().orc_topp(_i(out), _f(probs), B, V, topP, repeat_penalty, None, None, 0, _f(u), _i(ncand), _f(acc))
    return (out, ncand, acc) if return_details else out


def philox4x32_10(ctr, key):
    c = (C.c_uint32 * 4)(*ctr); k = (C.c_uint32 * 2)(*key); o = (C.c_uint32 * 4)()
    lib().orc_philox4x32_10(o, c, k)
    return [int(v) for v in o]


def philox_uniform(seed, seq, step):
    return float(lib().orc_philox_uniform(seed, seq, step))


def max_threads():
    return int(lib().orc_max_threads())


class OracleGPT:
    """The assembled token loop (Decoder.GPTDecode + GPT.RunForwardOnSingleDevice) on the CPU restatement."""

    def __init__(self, cfg, weights, max_pos=0, threads=1, faithful_cache=False):
        c = OrcConfig()
        c.L, c.d, c.H, c.Hkv, c.hd, c.F, c.V = cfg.L, cfg.d, cfg.H, cfg.kv_heads(), cfg.hd, cfg.F, cfg.V
        c.norm_type, c.act, c.pe_type, c.attn_type = int(cfg.norm), int(cfg.act), int(cfg.pe), int(cfg.attn)
        c.eps, c.rope_base = cfg.eps, cfg.rope_base
        c.ape_decode_pos0 = 1 if cfg.ape_decode_pos0 else 0
        c.max_pos, c.faithful_cache, c.threads = max_pos, 1 if faithful_cache else 0, threads
        c.n_experts, c.experts_per_token = getattr(cfg, "expertNum", 1), getattr(cfg, "expertsPerTokenFactor", 1)
        c.cross_attn = 1 if getattr(cfg, "cross_attn", False) else 0
        self.cfg = cfg
        self._h = lib().orc_create(C.byref(c))
        for name, w in weights.items():
            w = _c32(w)
            rows, cols = (w.shape if w.ndim == 2 else (1, w.size))
            if not lib().orc_set_weight(self._h, name.encode(), _f(w), rows, cols):
                raise KeyError("oracle does not know weight '%s'" % name)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_destroy(self._h)
            self._h = None

    def reset(self):
        lib().orc_reset(self._h)

    def set_encoder_output(self, enc, src_lens=None):
        """enc [B, S_src, d]: what the encoder handed to TransformerDecoder.Decode; src_lens: unpadded source lengths."""
        enc = _c32(enc)
        B, Ts = enc.shape[0], enc.shape[1]
        lens = None if src_lens is None else np.ascontiguousarray(src_lens, dtype=np.int32)
        if not lib().orc_set_encoder_output(self._h, _f(enc), _i(lens) if lens is not None else None, B, Ts):
            raise RuntimeError("oracle: the model has no cross-attention blocks or the shapes are wrong")

    def cache_len(self):
        return int(lib().orc_cache_len(self._h))

    def step(self, ids, temperature=1.0, blocked=()):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        B, S = ids.shape
        V = self.cfg.V
        logits = np.empty((B, V), dtype=np.float32)
        probs = np.empty((B, V), dtype=np.float32)
        bl = np.asarray(list(blocked), dtype=np.int32)
        ok = lib().orc_step(self._h, _i(ids), B, S, temperature, _i(bl) if bl.size else None, bl.size, _f(logits), _f(probs), None)
        if not ok:
            raise RuntimeError("oracle step failed (bad ids or cache/batch mismatch)")
        return logits, probs

    def generate(self, prompt, opts, uniforms=None, stop_on_eos=True, record=None):
        """prompt [B,S] -> ids [B,n]; opts is a DecodingOptions-like object; uniforms(step, b) -> u for Sampling."""
        prompt = np.asarray(prompt, dtype=np.int32)
        B, S = prompt.shape
        seqs = [list(map(int, r)) for r in prompt]
        sampling = int(opts.DecodingStrategy) == 1
        temp = opts.Temperature if sampling else 1.0
        blocked = opts.BlockedTokens or ()
        self.reset()
        out = []
        for i in range(S, opts.MaxTgtSentLength):
            step = i - S
            ids = prompt if step == 0 else np.array([[s[-1]] for s in seqs], dtype=np.int32)
            logits, probs = self.step(ids, temp, blocked)
            if sampling:
                u = np.array([uniforms(step, b) for b in range(B)], dtype=np.float32)
                nxt = topp(probs, opts.TopP, opts.RepeatPenalty, seqs, u)
            else:
                nxt = argmax(probs)
            if record is not None:
                record(step, logits, probs, nxt)
            for b in range(B):
                seqs[b].append(int(nxt[b]))
            out.append(nxt.copy())
            if stop_on_eos and all(s[-1] == 0 for s in seqs):
                break
        return np.stack(out, axis=1)
