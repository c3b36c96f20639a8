"""The give-up path of the persistent decode-step kernel, exercised without any fault: the host lowers the bound of the
kernel's dependency polls to one, so the first CTA that looks at a counter before its producers have finished gives
up.  The kernel must return (every CTA walks through the rest of its program without waiting), the call must fail with
a message, the engine must stay usable, and with the default bound restored the same prompt must give the same ids as
an engine that never failed.  Nothing here traps, faults or waits without a limit."""
import numpy as np
import pytest

from seq2seqsharp_b200 import _native as N
from seq2seqsharp_b200.gpt import DecodingOptions, GPT, synthetic_weights
from seq2seqsharp_b200.synthetic import prompt_ids
from tests.test_gpt_gpu import ARCHS

pytestmark = pytest.mark.gpu


@pytest.mark.timeout(300)
@pytest.mark.parametrize("cfg", [ARCHS[1], ARCHS[0]], ids=["fp16_tensor_core_consumers", "fp32_cuda_core_consumers"])
@pytest.mark.parametrize("call", ["decode", "step_host"])
def test_a_wait_that_runs_out_fails_the_call_and_leaves_the_engine_usable(cuda, cfg, call, monkeypatch):
    monkeypatch.setenv("TSB200_OWNER_MAXB", "1")    # one sequence on a persistent kernel (one-GPU fp16 engines default to one
    monkeypatch.setenv("TSB200_STACK_MAXB", "1")    # launch per operation): the kernels whose cross-CTA waits are bounded
    w = synthetic_weights(cfg, 21, std=0.04)
    prompt = prompt_ids(9, 1, 24, cfg.V)
    opts = DecodingOptions(MaxTgtSentLength=64, BlockedTokens=[0])
    gpt = GPT(cfg, max_batch=1, max_tokens=64)
    gpt.LoadWeights(w)
    first = gpt.Prefill(prompt, opts)
    good = gpt.Decode(6, opts)
    assert gpt.ProfileDecode(1, opts)["decode_stack"][1] == 1      # one sequence decodes through the persistent kernel
    # --- the wait runs out
    gpt.Reset()
    np.testing.assert_array_equal(gpt.Prefill(prompt, opts), first)
    gpt.SetWaitLimit(1)
    T_before = gpt.CacheLength()
    with pytest.raises(N.TSB200Error, match="gave up waiting"):
        if call == "decode":
            gpt.Decode(3, opts)
        else:
            gpt.StepHost(first, opts)
    assert gpt.CacheLength() == T_before       # the failed call committed nothing on the host side
    # --- and the engine is still good for ordinary calls
    gpt.SetWaitLimit(0)
    gpt.Reset()
    np.testing.assert_array_equal(gpt.Prefill(prompt, opts), first)
    np.testing.assert_array_equal(gpt.Decode(6, opts), good)
    gpt.close()
