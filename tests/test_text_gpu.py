"""File of lines in, file of lines out through the real engine (`GptTextRunner.Test`, the stand-in for the reference's
`GPT.Test(inputFile, outputFile, batchSize, ...)`, Tools/BaseSeq2SeqFramework.cs:987-992): every output line must be the
line's own tokens followed by what the same engine generates for that line alone, up to its first </s> or the length
limit, in input order - for whole batches, for batches of lines of different lengths, and through the slot scheduler."""
import numpy as np
import pytest

from seq2seqsharp_b200.gpt import (ActivateFuncEnums as A, DecodingOptions, DecodingStrategyEnums as DS, GPT, GPTConfig,
                                   MultiHeadAttentionTypeEnums as M, NormEnums as Nm, PositionEmbeddingEnums as P, synthetic_weights)
from seq2seqsharp_b200.text import GptTextRunner, Vocab

pytestmark = pytest.mark.gpu

CFG = GPTConfig(name="gqa_rope_fp32", L=2, d=128, H=4, Hkv=2, hd=32, F=256, V=120, norm=Nm.RMSNorm, act=A.SiLU, pe=P.RoPE, attn=M.GQA,
                dtype="float32")
MAX_TGT = 24


def _solo(g, ids, opts):
    out = g.RunForwardOnSingleDevice(np.asarray([ids], dtype=np.int32), opts, stop_on_eos=True)[0]
    out = [int(t) for t in out]
    return out[: out.index(0) + 1] if 0 in out else out


@pytest.mark.parametrize("use_scheduler", [False, True], ids=["batches", "slots"])
def test_file_to_file_matches_solo_runs(cuda, tmp_path, use_scheduler, monkeypatch):
    monkeypatch.setenv("TSB200_STACK", "0")   # one launch per operation in every run: a line's arithmetic does not depend on its batch
    vocab = Vocab(["w%d" % i for i in range(5, CFG.V - 1)] + ["tail"])          # 120 entries: ids 5..119
    assert vocab.Count == CFG.V
    w = synthetic_weights(CFG, 9, std=0.08, bias_std=0.02, max_pos=MAX_TGT + 10)
    rng = np.random.default_rng(21)
    lines = []
    for i in range(7):
        n = int(rng.integers(1, 9)) if i != 3 else 30                           # line 3 is cut to MaxSrcSentLength - 2 words
        lines.append(" ".join(vocab.GetString(int(t)) for t in rng.integers(5, CFG.V, size=n)))
    lines[5] = "unseen-word " + lines[5]                                         # maps to <unk>
    src, dst = tmp_path / "in.txt", tmp_path / "out.txt"
    src.write_text("\n".join(lines) + "\n", encoding="utf-8")
    opts = DecodingOptions(MaxSrcSentLength=12, MaxTgtSentLength=MAX_TGT, DecodingStrategy=DS.GreedySearch)
    g = GPT(CFG, max_batch=3, max_tokens=MAX_TGT + 16)
    g.LoadWeights(w)
    solo = GPT(CFG, max_batch=1, max_tokens=MAX_TGT + 16)
    solo.LoadWeights(w)
    run = GptTextRunner(g, vocab, opts, use_scheduler=use_scheduler, slots=3)
    got = run.Test(str(src), str(dst), batch_size=3)
    assert dst.read_text(encoding="utf-8").splitlines() == got and len(got) == len(lines)
    for line, out in zip(lines, got):
        words = ["<s>"] + line.split(" ")[: opts.MaxSrcSentLength - 2]
        ids = vocab.GetWordIndex([words])[0]
        want = words + vocab.ConvertIdsToString(_solo(solo, ids, opts))
        assert out.split(" ") == want, (line, out, want)
        assert len(want) <= MAX_TGT
    assert run.stats.lines == len(lines)
    g.CheckGuards()
    g.close()
    solo.close()
