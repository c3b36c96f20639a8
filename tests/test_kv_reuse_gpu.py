"""Parking and reusing KV caches across calls (GPT.cs:236-247 lookup, :312-328 store) and running a prompt suffix on
top of a cached head (Decoder.cs:661-697), on the GPU against the CPU oracle.

Tolerances: logits within 1e-3 (fp32) / 2e-2 (fp16) of the largest |logit| against the oracle; a cache that was
parked and restored must continue BIT-EXACTLY like the run that never left the device (same kernels, same inputs).
"""
import numpy as np
import pytest

from seq2seqsharp_b200 import _native as N
from seq2seqsharp_b200.gpt import GPT, KvCachePool, generate_with_pool
from seq2seqsharp_b200.synthetic import prompt_ids
from tests.golden.make_golden import CASES, SEED, case_inputs

pytestmark = pytest.mark.gpu


def rel_err(got, ref):
    return float(np.abs(got - ref).max() / max(1e-12, np.abs(ref).max()))


def tol_for(cfg):
    return 1e-3 if cfg.dtype == "float32" else 2e-2


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_restored_cache_continues_bit_exactly(cuda, case):
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    B, S = prompt.shape
    n1, n2 = 5, 6
    gpt = GPT(cfg, max_batch=B, max_tokens=opts.MaxTgtSentLength + 2)   # the APE table of the case has max_tokens + 2 rows
    gpt.LoadWeights(w)
    gpt.Reset()
    gpt.Prefill(prompt, opts)
    gpt.Decode(n1, opts)
    snap = gpt.CacheSnapshot()
    assert (snap.B, snap.T) == (B, S + n1)
    np.testing.assert_array_equal(snap.tokens[:, :S], prompt)
    want_ids = gpt.Decode(n2, opts)
    want_logits = gpt.Logits()[0]
    # something else uses the engine in between
    gpt.Reset()
    gpt.Prefill(prompt[:, ::-1].copy(), opts)
    gpt.Decode(3, opts)
    gpt.Reset()
    gpt.CacheRestore(snap)
    assert gpt.CacheLength() == S + n1
    got_ids = gpt.Decode(n2, opts)
    got_logits = gpt.Logits()[0]
    np.testing.assert_array_equal(got_ids, want_ids)
    np.testing.assert_array_equal(got_logits, want_logits)
    snap.close()
    gpt.close()


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
@pytest.mark.parametrize("suffix", [1, 4])
def test_prompt_suffix_on_cached_head_matches_oracle(cuda, oracle, case, suffix):
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    B, S = prompt.shape
    k = S - suffix
    sampling = int(opts.DecodingStrategy) == 1
    temp = opts.Temperature if sampling else 1.0
    orc = oracle.OracleGPT(cfg, w, max_pos=max_pos)
    orc.reset()
    orc.step(prompt[:, :k], temp, opts.BlockedTokens)
    lo, po = orc.step(prompt[:, k:], temp, opts.BlockedTokens)
    gpt = GPT(cfg, max_batch=B, max_tokens=opts.MaxTgtSentLength + 2)
    gpt.LoadWeights(w)
    gpt.Reset()
    gpt.Prefill(prompt[:, :k], opts)
    nxt = gpt.Extend(prompt[:, k:], opts)
    assert gpt.CacheLength() == S
    ld, pd = gpt.Logits()
    tol = tol_for(cfg)
    for b in range(B):
        assert rel_err(ld[b], lo[b]) <= tol
    if sampling:
        u = np.array([oracle.philox_uniform(opts.Seed, opts.SeqBase + b, 1) for b in range(B)], dtype=np.float32)
        hist = [list(map(int, prompt[b])) for b in range(B)]
        np.testing.assert_array_equal(nxt, oracle.topp(pd, opts.TopP, opts.RepeatPenalty, hist, u))
    else:
        np.testing.assert_array_equal(nxt, oracle.argmax(pd))
    # the loop goes on from the extended cache: one more step against the oracle fed with the device's id
    lo2, _ = orc.step(nxt[:, None], temp, opts.BlockedTokens)
    gpt.Decode(1, opts)
    ld2, _ = gpt.Logits()
    for b in range(B):
        assert rel_err(ld2[b], lo2[b]) <= tol
    gpt.close()


def test_one_parked_sequence_serves_a_batch(cuda, oracle):
    case = CASES[2]  # fp16 GQA RoPE greedy
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    head = prompt[:1, :10]
    B = 3
    tails = prompt_ids(SEED + 7, B, 5, cfg.V)
    gpt = GPT(cfg, max_batch=B, max_tokens=opts.MaxTgtSentLength + 2)
    gpt.LoadWeights(w)
    gpt.Reset()
    gpt.Prefill(head, opts)
    snap = gpt.CacheSnapshot()
    gpt.Reset()
    gpt.CacheRestore(snap, batch=B)
    # position T holds the pending id of the parked run; the tails are the text from there on
    gpt.Extend(tails, opts)
    ld, _ = gpt.Logits()
    orc = oracle.OracleGPT(cfg, w, max_pos=max_pos)
    for b in range(B):
        orc.reset()
        lo, _ = orc.step(np.concatenate([head, tails[b:b + 1]], axis=1), 1.0, opts.BlockedTokens)
        assert rel_err(ld[b], lo[0]) <= tol_for(cfg)
    snap.close()
    gpt.close()


def test_pool_round_trip_like_the_reference_cache(cuda):
    """Second request = first request's text + its output: the parked cache is picked up, one token is run
    (Decoder.cs:661-678) and the continuation equals the one a fresh engine computes from the whole text."""
    case = CASES[0]  # fp32 greedy
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    import dataclasses
    p1 = prompt[0]
    o1 = dataclasses.replace(opts, MaxTgtSentLength=len(p1) + 6)
    gpt = GPT(cfg, max_batch=1, max_tokens=opts.MaxTgtSentLength + 2)
    gpt.LoadWeights(w)
    pool = KvCachePool()
    out1 = generate_with_pool(gpt, pool, p1, o1, stop_on_eos=False)
    assert len(pool) == 1 and pool.misses == 1
    p2 = np.concatenate([p1, out1])
    o2 = dataclasses.replace(opts, MaxTgtSentLength=len(p2) + 6)
    out2 = generate_with_pool(gpt, pool, p2, o2, stop_on_eos=False)
    assert pool.hits == 1 and len(pool) == 1
    fresh = gpt.RunForwardOnSingleDevice(p2[None, :], o2, stop_on_eos=False)[0]
    np.testing.assert_array_equal(out2, fresh)
    # a request that shares only the head of a parked text still reuses it
    p3 = np.concatenate([p2[:len(p1) + 3], prompt_ids(SEED + 3, 1, 4, cfg.V)[0]])
    o3 = dataclasses.replace(opts, MaxTgtSentLength=len(p3) + 4)
    pool.clear()
    gpt.Reset()
    gpt.Prefill(p2[None, :len(p1) + 3], o3)
    pool.put(gpt.CacheSnapshot())
    out3 = generate_with_pool(gpt, pool, p3, o3, stop_on_eos=False)
    fresh3 = gpt.RunForwardOnSingleDevice(p3[None, :], o3, stop_on_eos=False)[0]
    np.testing.assert_array_equal(out3, fresh3)
    assert pool.hits == 2
    pool.clear()
    gpt.close()


def test_errors(cuda):
    case = CASES[0]
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    gpt = GPT(cfg, max_batch=2, max_tokens=24)
    gpt.LoadWeights(w)
    gpt.Reset()
    with pytest.raises(N.TSB200Error):
        gpt.Extend(prompt[:, :3], opts)          # nothing cached
    with pytest.raises(N.TSB200Error):
        gpt.CacheSnapshot()                      # nothing cached
    gpt.Prefill(prompt[:, :8], opts)
    with pytest.raises(N.TSB200Error):
        gpt.Extend(np.zeros((2, 3), dtype=np.int32), opts)   # batch differs from the cached one
    with pytest.raises(N.TSB200OutOfMemory):
        gpt.Extend(np.ones((1, 16), dtype=np.int32), opts)   # 8 + 16 positions do not fit 24
    snap = gpt.CacheSnapshot()
    other = GPT(CASES[2]["cfg"], max_batch=1, max_tokens=24)
    with pytest.raises(N.TSB200Error):
        other.CacheRestore(snap)                 # another model
    with pytest.raises(N.TSB200Error):
        gpt.CacheRestore(snap, batch=3)          # beyond the engine's batch capacity
    small = GPT(cfg, max_batch=1, max_tokens=8)
    with pytest.raises(N.TSB200OutOfMemory):
        small.CacheRestore(snap)                 # 8 cached positions need a longer cache
    small.close()
    other.close()
    snap.close()
    gpt.close()


def test_longer_prompt_on_a_used_engine(cuda):
    """A second request with a longer prompt grows the activation buffers; the captured decode step must follow."""
    import dataclasses
    case = CASES[0]
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    long_p = prompt[:, :12]
    short_p = prompt[:, :5]
    o = dataclasses.replace(opts, MaxTgtSentLength=20)
    used = GPT(cfg, max_batch=1, max_tokens=opts.MaxTgtSentLength + 2)
    used.LoadWeights(w)
    used.RunForwardOnSingleDevice(short_p, o, stop_on_eos=False)
    got = used.RunForwardOnSingleDevice(long_p, o, stop_on_eos=False)
    used.close()
    fresh = GPT(cfg, max_batch=1, max_tokens=opts.MaxTgtSentLength + 2)
    fresh.LoadWeights(w)
    want = fresh.RunForwardOnSingleDevice(long_p, o, stop_on_eos=False)
    fresh.close()
    np.testing.assert_array_equal(got, want)


def test_snapshot_of_a_cache_decoded_to_capacity(cuda):
    """Decoding may fill the cache to its last position (T == max_tokens); parking it then must work: the history has no
    slot left for the pending id, which the snapshot keeps separately."""
    case = CASES[0]
    cfg, w, prompt, opts, max_pos = case_inputs(case)
    S, cap = 6, 16
    gpt = GPT(cfg, max_batch=2, max_tokens=cap)
    gpt.LoadWeights(w)
    gpt.Reset()
    gpt.Prefill(prompt[:, :S], opts)
    ids = gpt.Decode(cap - S, opts)
    assert gpt.CacheLength() == cap
    snap = gpt.CacheSnapshot()
    assert snap.T == cap
    np.testing.assert_array_equal(snap.tokens[:, :S], prompt[:, :S])
    np.testing.assert_array_equal(snap.tokens[:, S + 1:cap], ids[:, :cap - S - 1])
    with pytest.raises(N.TSB200OutOfMemory):
        gpt.CacheRestore(snap)       # a full cache cannot take another step, so restoring it is refused as out of memory
    snap.close()
    gpt.close()
