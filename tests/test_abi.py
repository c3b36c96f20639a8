"""CPU tests of the drop-in boundary: the shared library loads, exports exactly what include/tsb200.h declares,
follows the 1/0 + thread-local last-error convention, and refuses to compute without a B200 (no CPU fallback)."""
import ctypes as C
import threading

import numpy as np
import pytest

from seq2seqsharp_b200 import _native as N


def test_header_symbols_are_exported(native):
    declared = N.declared_symbols()
    assert len(declared) >= 55
    missing = [s for s in declared if not hasattr(native, s)]
    assert not missing, "declared in tsb200.h but not exported: %s" % missing
    # and the binding table covers the header one-to-one
    assert sorted(native._tsb_signatures) == declared


def test_build_info_and_error_convention(native):
    assert native.TSB200_BuildInfo().decode().startswith("sm_100a;nvcc ")
    n = C.c_int(-1)
    ok = native.TSB200_DeviceCount(C.byref(n))
    assert ok in (0, 1) and n.value >= 0
    # a bad argument returns 0 and leaves a message; it never raises across the boundary
    assert native.TSB200_DeviceCount(None) == 0
    assert "null" in N.last_error()
    with pytest.raises(N.TSB200Error):
        N.call("TSB200_DeviceCount", None)


def test_last_error_is_thread_local(native):
    native.TSB200_DeviceCount(None)
    seen = {}

    def other():
        seen["msg"] = N.last_error()

    t = threading.Thread(target=other)
    t.start()
    t.join()
    assert seen["msg"] == "" and "null" in N.last_error()


def test_no_cpu_fallback_without_gpu(native):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the refusal path is exercised on CPU-only machines")
    assert native.TSB200_IsAvailable(0) == 0
    p = C.c_void_p()
    assert native.TSB200_Alloc(0, 1024, C.byref(p)) == 0
    assert "no CPU fallback" in N.last_error() or "CUDA" in N.last_error()
    cfg = N.GptConfig()
    cfg.L, cfg.d, cfg.H, cfg.Hkv, cfg.hd, cfg.F, cfg.V = 1, 64, 4, 4, 16, 64, 97
    cfg.max_batch, cfg.max_tokens, cfg.tp_size = 1, 16, 1
    h = C.c_void_p()
    assert native.TSB200_GptCreate(C.byref(cfg), C.byref(h)) == 0
    from seq2seqsharp_b200.gpt import GPT, GPTConfig
    with pytest.raises(N.TSB200Error):
        GPT(GPTConfig(L=1, d=64, H=4, hd=16, F=64, V=97), max_batch=1, max_tokens=16)


def test_workspace_queries_need_no_gpu(native):
    assert native.TSB200_TopPWorkspaceBytes(2, 1000) == 2 * 1000 * 20
    assert native.TSB200_LinearWorkspaceBytes(1, 4096, 4096) > 0
    assert native.TSB200_FlashDecodeWorkspaceBytes(1, 32, 128, 1024) > 0


def test_config_struct_layout_matches_header():
    # field order/size of the ctypes mirrors = the C structs (all 4-byte fields, no padding until the pointers)
    assert C.sizeof(N.GptConfig) == 24 * 4
    assert C.sizeof(N.Tensor) == 8 + 4 + 4 + 32 + 32
    assert N.DecodingOptionsC.blocked.offset == 16 and N.DecodingOptionsC.seed.offset == 32
