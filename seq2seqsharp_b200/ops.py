"""Python twin of TensorSharp.Ops (TensorSharp/Ops.cs:15-303) dispatching to the B200 backend.

In the reference every op goes Ops.X -> OpRegistry.Invoke(name, args) -> the backend method registered for the
storage type of the arguments (TensorSharp/OpRegistry.cs:46-64).  Here the tensors are torch CUDA tensors (used
only as device buffers with sizes and strides, exactly the fields of TensorSharp.Tensor) and each function calls
the C-ABI entry point that `B200BasicOps` binds for that op name.  `result=None` allocates the write target the way
TensorResultBuilder.GetWriteTarget does (TensorSharp/Core/TensorResultBuilder.cs:7-37).
"""
import ctypes as C

import torch

from . import _native as N

_DT = {torch.float32: N.F32, torch.float16: N.F16, torch.int32: N.I32, torch.float64: N.F64, torch.uint8: N.U8}


def desc(t):
    """TSB200Tensor descriptor of a torch CUDA tensor (a view: sizes, element strides, data pointer)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise N.TSB200Error("the B200 backend only accepts device tensors (no CPU fallback)")
    if t.dim() < 1 or t.dim() > 4:
        raise N.TSB200Error("tensors must have 1..4 dimensions")
    d = N.Tensor()
    d.data = t.data_ptr()
    d.dtype = _DT[t.dtype]
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.sizes[i] = t.size(i)
        d.strides[i] = t.stride(i)
    return d


def _ref(d):
    return C.byref(d) if d is not None else None


def _stream():
    """The caller's current torch stream.  On torch's legacy default stream (handle 0) the library would fall back to
    its own non-blocking stream, which does not order itself after torch's work, so pending torch work is waited for
    first."""
    h = torch.cuda.current_stream().cuda_stream
    if h == 0:
        torch.cuda.synchronize()
        return None
    return C.c_void_p(h)


def _dev(t):
    return t.device.index or 0


def _target(result, like, sizes=None, dtype=None):
    if result is not None:
        return result
    return torch.empty(tuple(sizes if sizes is not None else like.shape), dtype=dtype or like.dtype, device=like.device)


class Ops:
    """Static facade with the reference's op names."""

    @staticmethod
    def Copy(result, src):
        N.call("TSB200_Copy", _dev(src), _ref(desc(result)), _ref(desc(src)), _stream())
        return result

    @staticmethod
    def Fill(result, value):
        N.call("TSB200_Fill", _dev(result), _ref(desc(result)), float(value), _stream())
        return result

    @staticmethod
    def AsContiguous(src):
        if src.is_contiguous():
            return src
        r = torch.empty(tuple(src.shape), dtype=src.dtype, device=src.device)
        return Ops.Copy(r, src)

    @staticmethod
    def Addmm(result, beta, src, alpha, m1, m2):
        r = _target(result, src)
        N.call("TSB200_Addmm", _dev(src), _ref(desc(r)), float(beta), _ref(desc(src)), float(alpha), _ref(desc(m1)),
               _ref(desc(m2)), _stream())
        return r

    @staticmethod
    def AddmmBatch(result, beta, src, alpha, m1, m2):
        r = _target(result, src)
        N.call("TSB200_AddmmBatch", _dev(src), _ref(desc(r)), float(beta), _ref(desc(src)), float(alpha),
               _ref(desc(m1)), _ref(desc(m2)), _stream())
        return r

    @staticmethod
    def LayerNorm(result, src, alpha, beta, eps=1e-9):
        r = _target(result, src)
        N.call("TSB200_LayerNorm", _dev(src), _ref(desc(r)), _ref(desc(src)), _ref(desc(alpha)), _ref(desc(beta)),
               float(eps), _stream())
        return r

    @staticmethod
    def RMSNorm(result, src, alpha, beta, eps=1e-9):
        r = _target(result, src)
        N.call("TSB200_RMSNorm", _dev(src), _ref(desc(r)), _ref(desc(src)), _ref(desc(alpha)), _ref(desc(beta)),
               float(eps), _stream())
        return r

    @staticmethod
    def RoPE(result, src, seqLen, rowOffset, base=None):
        r = _target(result, src)
        if base is None:
            N.call("TSB200_RoPE", _dev(src), _ref(desc(r)), _ref(desc(src)), int(seqLen), int(rowOffset), _stream())
        else:
            N.call("TSB200_RoPEEx", _dev(src), _ref(desc(r)), _ref(desc(src)), int(seqLen), int(rowOffset),
                   float(base), _stream())
        return r

    @staticmethod
    def Softmax(result, src):
        r = _target(result, src)
        N.call("TSB200_Softmax", _dev(src), _ref(desc(r)), _ref(desc(src)), _stream())
        return r

    @staticmethod
    def IndexSelect(result, src, indice, isAdd=False):
        r = _target(result, src, sizes=(indice.numel(), src.shape[1]))
        N.call("TSB200_IndexSelect", _dev(src), _ref(desc(r)), _ref(desc(src)), _ref(desc(indice)), int(isAdd),
               _stream())
        return r

    @staticmethod
    def Add(result, lhs, rhs):
        r = _target(result, lhs)
        if isinstance(rhs, (int, float)):
            raise N.TSB200Error("Add with a scalar is not on the GPT decode path")
        N.call("TSB200_Add", _dev(lhs), _ref(desc(r)), _ref(desc(lhs)), _ref(desc(rhs)), _stream())
        return r

    @staticmethod
    def Mul(result, lhs, rhs):
        r = _target(result, lhs)
        if isinstance(rhs, (int, float)):
            N.call("TSB200_MulScalar", _dev(lhs), _ref(desc(r)), _ref(desc(lhs)), float(rhs), _stream())
        else:
            N.call("TSB200_Mul", _dev(lhs), _ref(desc(r)), _ref(desc(lhs)), _ref(desc(rhs)), _stream())
        return r

    @staticmethod
    def Div(result, lhs, rhs):
        r = _target(result, lhs)
        N.call("TSB200_DivScalar", _dev(lhs), _ref(desc(r)), _ref(desc(lhs)), float(rhs), _stream())
        return r

    @staticmethod
    def Relu(result, src):
        r = _target(result, src)
        N.call("TSB200_Relu", _dev(src), _ref(desc(r)), _ref(desc(src)), _stream())
        return r

    @staticmethod
    def SiLU(result, src):
        r = _target(result, src)
        N.call("TSB200_SiLU", _dev(src), _ref(desc(r)), _ref(desc(src)), _stream())
        return r

    @staticmethod
    def LeakyReLU(result, src):
        r = _target(result, src)
        N.call("TSB200_LeakyReLU", _dev(src), _ref(desc(r)), _ref(desc(src)), _stream())
        return r

    @staticmethod
    def Float2Half(result, src):
        r = _target(result, src, dtype=torch.float16)
        N.call("TSB200_Float2Half", _dev(src), _ref(desc(r)), _ref(desc(src)), _stream())
        return r

    @staticmethod
    def Half2Float(result, src):
        r = _target(result, src, dtype=torch.float32)
        N.call("TSB200_Half2Float", _dev(src), _ref(desc(r)), _ref(desc(src)), _stream())
        return r

    @staticmethod
    def Argmax(result, src, dimension):
        if dimension < 0:
            dimension += src.dim()
        sizes = list(src.shape)
        sizes[dimension] = 1
        r = _target(result, src, sizes=sizes)
        N.call("TSB200_Argmax", _dev(src), _ref(desc(r)), _ref(desc(src)), int(dimension), _stream())
        return r

    @staticmethod
    def BuildTriMask(result, value, maskedValue):
        N.call("TSB200_BuildTriMask", _dev(result), _ref(desc(result)), float(value), float(maskedValue), _stream())
        return result

    @staticmethod
    def BuildSelfTriMask(result, originalLengths, paddedSeqLen, value, maskedValue):
        N.call("TSB200_BuildSelfTriMask", _dev(result), _ref(desc(result)), _ref(desc(originalLengths)),
               int(paddedSeqLen), float(value), float(maskedValue), _stream())
        return result

    # ---- device replacement of the host loop ComputeGraphTensor.TopPSample (ComputeGraphTensor.cs:2305-2403)
    @staticmethod
    def TopPSample(probs, topP, repeatPenalty, decodedSequences, u):
        """probs [rows, V] float32; decodedSequences: list of id lists (or None); u: [rows] float32 uniform draws."""
        rows, V = probs.shape
        dev = probs.device
        out = torch.empty(rows, dtype=torch.int32, device=dev)
        ws_bytes = N.lib().TSB200_TopPWorkspaceBytes(rows, V)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        hist = hist_len = None
        stride = 0
        if decodedSequences is not None:
            stride = max(1, max(len(s) for s in decodedSequences))
            h = torch.zeros((rows, stride), dtype=torch.int32)
            for i, s in enumerate(decodedSequences):
                if len(s):
                    h[i, :len(s)] = torch.tensor(s, dtype=torch.int32)
            hist = h.to(dev)
            hist_len = torch.tensor([len(s) for s in decodedSequences], dtype=torch.int32, device=dev)
        u = u.to(device=dev, dtype=torch.float32).contiguous()
        p = probs.contiguous()
        N.call("TSB200_TopPSample", _dev(probs), out.data_ptr(), p.data_ptr(), rows, V, float(topP),
               float(repeatPenalty), hist.data_ptr() if hist is not None else None,
               hist_len.data_ptr() if hist_len is not None else None, stride, u.data_ptr(), ws.data_ptr(), ws_bytes,
               _stream())
        return out

    @staticmethod
    def PhiloxUniform(n, seed, seq_first, step, device="cuda:0"):
        u = torch.empty(n, dtype=torch.float32, device=device)
        N.call("TSB200_PhiloxUniform", u.device.index or 0, u.data_ptr(), n, seed, seq_first, step, _stream())
        return u
