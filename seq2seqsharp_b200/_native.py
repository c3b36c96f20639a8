"""ctypes binding of libtsb200.so — the Python twin of the C# P/Invoke class a maintainer would add as
TensorSharp.B200/B200Native.cs (modelled on TensorSharp.GGML/GgmlNative.cs:161-331).

The library is loaded from the package directory.  There is no fallback: if the shared object is missing or a
call fails, a TSB200Error is raised (the C# binding raises InvalidOperationException / OutOfMemoryException in
the same places, GgmlNative.cs:471-479).
"""
import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
# TSB200_LIB: another build of the library (e.g. libtsb200_checked.so from `python -m seq2seqsharp_b200.build --checked`)
LIB_PATH = os.environ.get("TSB200_LIB") or os.path.join(_HERE, "libtsb200.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "tsb200.h")

F32, F16, F64, I32, U8 = 0, 1, 2, 3, 4
ACT_NONE, ACT_RELU, ACT_SILU, ACT_LEAKYRELU, ACT_GLU_NOACT, ACT_SWIGLU, ACT_GELU = -1, 0, 1, 2, 3, 4, 5


class TSB200Error(RuntimeError):
    pass


class TSB200OutOfMemory(TSB200Error, MemoryError):
    """Raised when the native error message starts with 'OOM:' (the C# binding maps it to OutOfMemoryException,
    which GPT.RunForwardOnSingleDevice catches: Seq2SeqSharp/Applications/GPT.cs:269)."""


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("sizes", C.c_int64 * 4), ("strides", C.c_int64 * 4)]


class GptConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("L", "d", "H", "Hkv", "hd", "F", "V", "norm_type", "act", "pe_type",
                                          "attn_type", "dtype")] + \
               [("eps", C.c_float), ("rope_base", C.c_float)] + \
               [(n, C.c_int32) for n in ("ape_decode_pos0", "max_batch", "max_tokens", "device", "tp_rank", "tp_size", "n_experts",
                                         "experts_per_token", "cross_attn", "max_src_tokens")]


class DecodingOptionsC(C.Structure):
    _fields_ = [("strategy", C.c_int32), ("topP", C.c_float), ("temperature", C.c_float),
                ("repeatPenalty", C.c_float), ("blocked", C.POINTER(C.c_int32)), ("n_blocked", C.c_int32),
                ("seed", C.c_uint64), ("seq_base", C.c_uint64)]


_lib = None


def declared_symbols():
    """Every TSB200_* function name declared in include/tsb200.h (without the development-build block)."""
    with open(HEADER_PATH) as fh:
        text = fh.read()
    text = re.sub(r"#ifdef TSB200_TRACE.*?#endif", "", text, flags=re.S)
    return sorted(set(re.findall(r"TSB200_API\s+[\w\s\*]+?\b(TSB200_\w+)\s*\(", text)))


def lib():
    """Loads libtsb200.so (once).  Raises TSB200Error when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TSB200Error("libtsb200.so is not built (%s); run `python -m seq2seqsharp_b200.build`. "
                          "There is no CPU fallback." % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    vp, i32, i64, f32, u64, u32 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint64, C.c_uint32
    TP = C.POINTER(Tensor)
    sig = {
        "TSB200_GetLastError": (C.c_char_p, []),
        "TSB200_IsAvailable": (i32, [i32]),
        "TSB200_DeviceCount": (i32, [C.POINTER(i32)]),
        "TSB200_BuildInfo": (C.c_char_p, []),
        "TSB200_LaunchCount": (i32, [i32, C.POINTER(i64)]),
        "TSB200_Alloc": (i32, [i32, i64, C.POINTER(vp)]),
        "TSB200_Free": (i32, [i32, vp]),
        "TSB200_MemcpyH2D": (i32, [i32, vp, vp, i64, vp]),
        "TSB200_MemcpyD2H": (i32, [i32, vp, vp, i64, vp]),
        "TSB200_MemcpyD2D": (i32, [i32, vp, vp, i64, vp]),
        "TSB200_MemcpyPeer": (i32, [i32, vp, i32, vp, i64]),
        "TSB200_Synchronize": (i32, [i32, vp]),
        "TSB200_MemoryInfo": (i32, [i32, C.POINTER(i64), C.POINTER(i64)]),
        "TSB200_Copy": (i32, [i32, TP, TP, vp]),
        "TSB200_Fill": (i32, [i32, TP, f32, vp]),
        "TSB200_Addmm": (i32, [i32, TP, f32, TP, f32, TP, TP, vp]),
        "TSB200_AddmmBatch": (i32, [i32, TP, f32, TP, f32, TP, TP, vp]),
        "TSB200_LayerNorm": (i32, [i32, TP, TP, TP, TP, f32, vp]),
        "TSB200_RMSNorm": (i32, [i32, TP, TP, TP, TP, f32, vp]),
        "TSB200_RoPE": (i32, [i32, TP, TP, i32, i32, vp]),
        "TSB200_RoPEEx": (i32, [i32, TP, TP, i32, i32, f32, vp]),
        "TSB200_Softmax": (i32, [i32, TP, TP, vp]),
        "TSB200_IndexSelect": (i32, [i32, TP, TP, TP, i32, vp]),
        "TSB200_Add": (i32, [i32, TP, TP, TP, vp]),
        "TSB200_Mul": (i32, [i32, TP, TP, TP, vp]),
        "TSB200_MulScalar": (i32, [i32, TP, TP, f32, vp]),
        "TSB200_DivScalar": (i32, [i32, TP, TP, f32, vp]),
        "TSB200_Relu": (i32, [i32, TP, TP, vp]),
        "TSB200_SiLU": (i32, [i32, TP, TP, vp]),
        "TSB200_LeakyReLU": (i32, [i32, TP, TP, vp]),
        "TSB200_Float2Half": (i32, [i32, TP, TP, vp]),
        "TSB200_Half2Float": (i32, [i32, TP, TP, vp]),
        "TSB200_Argmax": (i32, [i32, TP, TP, i32, vp]),
        "TSB200_BuildTriMask": (i32, [i32, TP, f32, f32, vp]),
        "TSB200_BuildSelfTriMask": (i32, [i32, TP, TP, i32, f32, f32, vp]),
        "TSB200_TopPWorkspaceBytes": (i64, [i32, i32]),
        "TSB200_TopPSample": (i32, [i32, vp, vp, i32, i32, f32, f32, vp, vp, i32, vp, vp, i64, vp]),
        "TSB200_TopPSampleStatic": (i32, [i32, vp, vp, i32, i32, f32, f32, vp, vp, i32, vp, vp]),
        "TSB200_PhiloxUniform": (i32, [i32, vp, i32, u64, u64, u32, vp]),
        "TSB200_LinearBiasAct": (i32, [i32, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, i64, vp]),
        "TSB200_LinearWorkspaceBytes": (i64, [i32, i32, i32]),
        "TSB200_PackedWeightBytes": (i64, [i32, i32, i32]),
        "TSB200_PackWeight": (i32, [i32, i32, vp, vp, i32, i32, i32, vp]),
        "TSB200_LinearPackedWorkspaceBytes": (i64, [i32, i32, i32, i32]),
        "TSB200_LinearPacked": (i32, [i32, i32, vp, vp, vp, vp, vp, vp, i32, f32, vp, vp, vp, i32, i32, i32, i32, vp, i64, vp]),
        "TSB200_NormResidual": (i32, [i32, i32, vp, vp, vp, vp, vp, i32, f32, i32, i32, vp]),
        "TSB200_RopeAppend": (i32, [i32, i32, vp, vp, vp, i64, i64, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp]),
        "TSB200_FlashDecodeWorkspaceBytes": (i64, [i32, i32, i32, i32]),
        "TSB200_FlashDecode": (i32, [i32, i32, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, vp, i64, vp]),
        "TSB200_PrefillAttention": (i32, [i32, i32, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp]),
        "TSB200_SoftmaxArgmax": (i32, [i32, vp, vp, vp, i32, i32, f32, vp, i32, vp]),
        "TSB200_GptCreate": (i32, [C.POINTER(GptConfig), C.POINTER(vp)]),
        "TSB200_GptDestroy": (i32, [vp]),
        "TSB200_GptSetWeight": (i32, [vp, C.c_char_p, vp, i32, i64, i64, i32]),
        "TSB200_GptGetWeightPtr": (i32, [vp, C.c_char_p, C.POINTER(vp), C.POINTER(i64), C.POINTER(i64)]),
        "TSB200_GptFillSynthetic": (i32, [vp, u64, f32, f32]),
        "TSB200_CommGetUniqueId": (i32, [vp]),
        "TSB200_CommInitRank": (i32, [vp, i32, i32, i32, C.POINTER(vp)]),
        "TSB200_CommPeerExport": (i32, [vp, i64, vp]),
        "TSB200_CommPeerImport": (i32, [vp, vp, i32]),
        "TSB200_CommDestroy": (i32, [vp]),
        "TSB200_CommPeerClose": (i32, [vp]),
        "TSB200_GptTpClose": (i32, [vp]),
        "TSB200_AllReduceSumF32": (i32, [vp, vp, i64, vp]),
        "TSB200_GptTpExport": (i32, [vp, vp]),
        "TSB200_GptTpImport": (i32, [vp, vp, i32]),
        "TSB200_GptSetComm": (i32, [vp, vp]),
        "TSB200_GptReset": (i32, [vp]),
        "TSB200_GptSetWaitLimit": (i32, [vp, i32]),
        "TSB200_OwnerLayoutSelfTest": (i32, [i32] * 9),
        "TSB200_GptPrefill": (i32, [vp, vp, i32, i32, C.POINTER(DecodingOptionsC), vp]),
        "TSB200_GptDecode": (i32, [vp, i32, C.POINTER(DecodingOptionsC), i32, vp, C.POINTER(i32)]),
        "TSB200_GptGetLogits": (i32, [vp, vp, vp]),
        "TSB200_GptCacheLength": (i32, [vp, C.POINTER(i32)]),
        "TSB200_GptDecodePath": (i32, [vp, C.POINTER(i32)]),
        "TSB200_GptCheckGuards": (i32, [vp]),
        "TSB200_GptCacheLengths": (i32, [vp, vp, i32]),
        "TSB200_GptPrefillRagged": (i32, [vp, vp, vp, i32, i32, C.POINTER(DecodingOptionsC), vp]),
        "TSB200_GptSlotSnapshot": (i32, [vp, i32, C.POINTER(vp)]),
        "TSB200_GptSlotRestore": (i32, [vp, vp, i32]),
        "TSB200_GptSlotReset": (i32, [vp, i32]),
        "TSB200_GptSetPerSequenceState": (i32, [vp, i32]),
        "TSB200_GptSlotExtend": (i32, [vp, i32, vp, i32, C.POINTER(DecodingOptionsC), vp]),
        "TSB200_GptExtend": (i32, [vp, vp, i32, i32, C.POINTER(DecodingOptionsC), vp]),
        "TSB200_GptCacheSnapshot": (i32, [vp, C.POINTER(vp)]),
        "TSB200_GptCacheSnapshotInfo": (i32, [vp, C.POINTER(i32), C.POINTER(i32), C.POINTER(i64), vp]),
        "TSB200_GptCacheRestore": (i32, [vp, vp, i32]),
        "TSB200_GptCacheSnapshotFree": (i32, [vp]),
        "TSB200_GptLastTiming": (i32, [vp, C.POINTER(f32), C.POINTER(i64)]),
        "TSB200_GptStream": (i32, [vp, C.POINTER(vp)]),
        "TSB200_GptStepHost": (i32, [vp, vp, C.POINTER(DecodingOptionsC), vp]),
        "TSB200_GptSetEncoderOutput": (i32, [vp, vp, i32, i32, vp, i32, i32, i32]),
        "TSB200_GptBeamCandidates": (i32, [vp, i32, C.POINTER(DecodingOptionsC), vp, vp, vp]),
        "TSB200_GptBeamCopy": (i32, [vp, vp, vp, i32]),
        "TSB200_GptEnableStepTiming": (i32, [vp, i32]),
        "TSB200_GptGetStepTimes": (i32, [vp, vp, i32, C.POINTER(i32)]),
        "TSB200_GptProfileDecode": (i32, [vp, i32, C.POINTER(DecodingOptionsC), vp, vp, i32]),
        "TSB200_GptStepBytes": (i32, [vp, i32, i32, C.POINTER(i64)]),
        "TSB200_FillSynthetic": (i32, [i32, vp, i32, i64, u64, u64, f32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    L._tsb_signatures = sig
    _lib = L
    return L


def last_error():
    msg = lib().TSB200_GetLastError()
    return msg.decode("utf-8", "replace") if msg else ""


def check(result, op):
    """CheckResult of the C# binding: 0 -> exception carrying the thread-local native message."""
    if result:
        return
    msg = last_error()
    if msg.startswith("OOM:"):
        raise TSB200OutOfMemory("native %s failed. %s" % (op, msg))
    raise TSB200Error("native %s failed. %s" % (op, msg or "unknown native error"))


def call(name, *args):
    check(getattr(lib(), name)(*args), name)
