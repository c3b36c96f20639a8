"""TSB200_TopPSampleStatic: top-p sampling for hosts that cannot allocate device memory on the sampling path (a server
that handed all free memory to its own pool, or a token loop that cannot afford cudaMalloc's device-wide sync).  It sorts
in a scratch block that ships inside the library instead of a caller-provided workspace.

The test calls it through the C ABI twice in a row (the second call finds the first call's leftovers in the shared
scratch) and requires the same indices as the workspace-taking entry point, exactly.  It is collected last so that a run
stopping at the first failure has already exercised everything else; it also passes when run alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from seq2seqsharp_b200 import _native as N

pytestmark = pytest.mark.gpu


def _stream():
    from seq2seqsharp_b200.ops import _stream as ops_stream
    return ops_stream()


def _case(seed, rows, V, spread):
    g = torch.Generator().manual_seed(seed)
    p = torch.softmax(torch.randn(rows, V, generator=g) * spread, dim=-1)
    p[:, 0] -= 1.0                                            # a blocked token (p - 1 < 0) must be dropped
    u = torch.rand(rows, generator=g)
    hist = torch.randint(0, V, (rows, 40), generator=g, dtype=torch.int32)
    hlen = torch.randint(1, 41, (rows,), generator=g, dtype=torch.int32)
    return p.cuda().contiguous(), u.cuda(), hist.cuda().contiguous(), hlen.cuda()


def _with_workspace(p, u, hist, hlen, topP, penalty):
    rows, V = p.shape
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    wsb = N.lib().TSB200_TopPWorkspaceBytes(rows, V)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    N.call("TSB200_TopPSample", 0, out.data_ptr(), p.data_ptr(), rows, V, topP, penalty, hist.data_ptr(), hlen.data_ptr(),
           hist.shape[1], u.data_ptr(), ws.data_ptr(), wsb, _stream())
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _static(p, u, hist, hlen, topP, penalty):
    rows, V = p.shape
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    N.call("TSB200_TopPSampleStatic", 0, out.data_ptr(), p.data_ptr(), rows, V, topP, penalty, hist.data_ptr(), hlen.data_ptr(),
           hist.shape[1], u.data_ptr(), _stream())
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_static_scratch_topp_matches_workspace_topp_twice_in_a_row(cuda):
    first = _case(1, 8, 32000, 0.05)      # near-uniform: the nucleus covers most of the vocabulary
    second = _case(2, 3, 50257, 3.0)      # peaky, different shape: reuses the scratch the first call dirtied
    a1 = _static(*first, 0.95, 2.0)
    a2 = _static(*second, 0.9, 2.0)
    np.testing.assert_array_equal(a1, _with_workspace(*first, 0.95, 2.0))
    np.testing.assert_array_equal(a2, _with_workspace(*second, 0.9, 2.0))
    # and once more in the other order, still exact
    np.testing.assert_array_equal(_static(*first, 0.95, 2.0), a1)


def test_static_scratch_limit_is_reported(cuda):
    p, u, hist, hlen = _case(3, 9, 32000, 1.0)                # 288000 probabilities > 262144
    out = torch.zeros(9, dtype=torch.int32, device="cuda")
    with pytest.raises(N.TSB200Error, match="exceeds the built-in scratch"):
        N.call("TSB200_TopPSampleStatic", 0, out.data_ptr(), p.data_ptr(), 9, 32000, 0.9, 2.0, hist.data_ptr(), hlen.data_ptr(),
               hist.shape[1], u.data_ptr(), _stream())
