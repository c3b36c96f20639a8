"""The -DTSB200_CHECKED build of the library (device-side index / capacity checks that record a code and skip the access):
a normal prefill + decode runs clean through it, a recorded code fails the next engine call with its number, and the call
after that works again.  Runs in a child process because a process holds one build of the library."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import ctypes as C, sys
    import numpy as np
    from seq2seqsharp_b200 import _native as N
    from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, DecodingOptions, GPT, GPTConfig, MultiHeadAttentionTypeEnums as M,
                                       NormEnums as Nm, PositionEmbeddingEnums as P, synthetic_weights)
    assert N.LIB_PATH.endswith("libtsb200_checked.so"), N.LIB_PATH
    lib = N.lib()
    for dtype in ("float32", "float16"):
        cfg = GPTConfig(L=2, d=128, H=4, Hkv=2, hd=32, F=256, V=301, norm=Nm.RMSNorm, act=A.SiLU, pe=P.RoPE, attn=M.GQA, dtype=dtype)
        g = GPT(cfg, max_batch=3, max_tokens=48)
        g.LoadWeights(synthetic_weights(cfg, 5, std=0.08))
        opts = DecodingOptions(MaxTgtSentLength=40)
        ids = g.RunForwardOnSingleDevice(np.arange(1, 16, dtype=np.int32).reshape(3, 5), opts, stop_on_eos=False)
        assert ids.shape == (3, 35)
        g.Reset()
        g.PrefillRagged([[1, 2, 3, 4], [5, 6], [7]], opts)
        g.Decode(6, opts)                                   # per-sequence lengths: every check sees per-row state
        lib.TSB200_DebugCheckedSelfTest.argtypes = [C.c_int, C.c_int]
        assert lib.TSB200_DebugCheckedSelfTest(0, 0x1ff) == 1
        try:
            g.Decode(2, opts)
            raise SystemExit("a recorded device-side check did not fail the call")
        except N.TSB200Error as e:
            assert "device-side check 0x1ff" in str(e), str(e)
        g.Reset()
        g.Prefill(np.arange(1, 7, dtype=np.int32).reshape(3, 2), opts)
        g.Decode(3, opts)                                   # the word was cleared: the engine works again
        g.CheckGuards()
        g.close()
    print("checked build ok")
""")


def test_checked_build_runs_clean_and_reports_a_recorded_code(cuda):
    from seq2seqsharp_b200 import build
    lib = build.build(variant="checked")
    env = dict(os.environ, TSB200_LIB=lib, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "checked build ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
