"""Text front end (vocabulary, SentencePiece wrapper, line reader / writer, the file-to-file runner) on the CPU, with a
stand-in engine.  Reference behaviour: Utils/Vocab.cs, Utils/Misc.cs:83-91, Corpus/SntBatchStreamReader.cs,
Corpus/SntBatchStreamWriter.cs, Corpus/SeqCorpusBatch.cs:29-47, Tools/BaseSeq2SeqFramework.cs:73-87, GPT.cs:182-200."""
import os
import random

import numpy as np
import pytest

from seq2seqsharp_b200.gpt import DecodingOptions
from seq2seqsharp_b200.text import (AppendNewBatch, BuildInTokens, GptTextRunner, RemoveDuplicatedEOS, SENTTAGS, SentencePiece,
                                    SntBatchStreamReader, SntBatchStreamWriter, Vocab)


def test_vocab_file_rules(tmp_path):
    p = tmp_path / "v.txt"
    p.write_text("hello\t17\n</s>\t0\nworld\n<unk>\nfoo\tbar\tbaz\nlast\n", encoding="utf-8")
    v = Vocab.from_file(str(p))
    # built-in tokens keep ids 0..4 and are skipped in the file; words follow in file order
    assert [v.GetString(i) for i in range(5)] == ["</s>", "<s>", "<unk>", "[SEP]", "[CLS]"]
    assert [v.GetWordIndex(w) for w in ("hello", "world", "foo", "last")] == [5, 6, 7, 8]
    assert v.Count == 10 and v.GetString(9) == "[PAD_0]"          # nine entries -> one pad token for an even table
    assert v.GetWordIndex("nope") == SENTTAGS.UNK and v.GetString(1234) == BuildInTokens.UNK
    assert v.GetWordIndex([["<s>", "hello", "nope"], []]) == [[1, 5, 2], []]
    assert v.ConvertIdsToString([[5, 0], [77]]) == [["hello", "</s>"], ["<unk>"]]
    assert v.ConvertIdsToString([6, 8]) == ["world", "last"]
    out = tmp_path / "dump.txt"
    v.DumpVocab(str(out))
    lines = out.read_text(encoding="utf-8").splitlines()
    assert lines[0] == "</s>\t0" and lines[5] == "hello\t5" and len(lines) == 10
    # an even table stays as it is; a dumped table loads back to the same ids
    v2 = Vocab.from_file(str(out))
    assert v2.Count == 10 and v2.GetWordIndex("last") == 8


def test_vocab_from_model_table_and_ignore_case():
    v = Vocab.from_index_table(["</s>", "<s>", "<unk>", "[SEP]", "[CLS]", "Alpha", "beta"], ignore_case=True)
    assert v.Count == 7                        # a stored table is taken as it is: nothing skipped, nothing appended
    assert v.GetWordIndex("alpha") == 5 and v.GetWordIndex("BETA") == 6 and v.GetString(5) == "Alpha"


def test_append_new_batch_truncates_to_max_minus_two():
    b = []
    AppendNewBatch(b, "  a b c d e f  ", 6)
    AppendNewBatch(b, "x", 6)
    AppendNewBatch(b, "a  b", 6)           # split at single blanks: an empty token stays, as in the reference
    assert b == [["a", "b", "c", "d"], ["x"], ["a", "", "b"]]


def test_reader_batches_in_order_with_bos(tmp_path):
    p = tmp_path / "in.txt"
    p.write_text("one two three\n<s> already there\n\nlast line here now\n", encoding="utf-8")
    with SntBatchStreamReader(str(p), 3, 5) as r:
        i0, b0 = r.GetNextBatch()
        i1, b1 = r.GetNextBatch()
        i2, b2 = r.GetNextBatch()
    assert (i0, i1, i2) == (0, 3, -1) and b2 is None
    assert b0 == [["<s>", "one", "two", "three"], ["<s>", "already", "there"], ["<s>", ""]]
    assert b1 == [["<s>", "last", "line", "here"]]            # cut to 5 - 2 tokens, then <s> in front


def test_remove_duplicated_eos():
    s = [["a", "</s>", "b", "</s>"], ["a", "b"], ["</s>"]]
    RemoveDuplicatedEOS(s)
    assert s == [["a", "</s>"], ["a", "b"], ["</s>"]]


def test_writer_restores_input_order(tmp_path):
    p = tmp_path / "out.txt"
    w = SntBatchStreamWriter(str(p))
    w.WriteResults(2, [[["c"], ["d", "e"]]])                  # lines 2 and 3 arrive first: nothing can be written yet
    assert w.lines == []
    w.WriteResults(0, [[["a"], ["b"]], [["a2"], ["b2"]]])     # two beams: joined by a tab
    assert w.lines == ["a\ta2", "b\tb2", "c", "d e"]
    w.WriteResults(4, [[["f"]]])
    w.Close()
    assert p.read_text(encoding="utf-8").splitlines() == ["a\ta2", "b\tb2", "c", "d e", "f"]


@pytest.fixture(scope="module")
def spm_model(tmp_path_factory):
    spm = pytest.importorskip("sentencepiece")
    d = tmp_path_factory.mktemp("spm")
    rnd = random.Random(3)
    words = ["hello", "world", "the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "token", "loop", "decoder", "cache"]
    corpus = d / "corpus.txt"
    corpus.write_text("\n".join(" ".join(rnd.choice(words) for _ in range(rnd.randint(3, 9))) for _ in range(500)), encoding="utf-8")
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(d / "m"), vocab_size=80, model_type="bpe", minloglevel=2)
    return str(d / "m.model")


def test_sentencepiece_round_trip(spm_model):
    sp = SentencePiece(spm_model)
    enc = sp.Encode("the quick brown fox")
    assert enc.startswith("▁") and " " in enc
    assert sp.Decode(enc) == "the quick brown fox"
    assert sp.Decode(["<s>"] + enc.split(" ") + ["</s>"]) == "the quick brown fox"   # control pieces print as nothing
    assert sp.Encode("The QUICK", toLower=True) == sp.Encode("the quick")


class _EchoEngine:
    """Stands in for the GPT engine: the next id of a sequence is (last id + 1) mod V, id 7 is followed by </s>."""

    def __init__(self, V=12):
        self.V, self.seqs, self.calls = V, [], []

    def _next(self, last):
        return 0 if last == 7 else (last + 1) % self.V

    def Reset(self):
        self.seqs = []

    def Prefill(self, ids, opts):
        self.calls.append(("prefill", np.asarray(ids).shape))
        self.seqs = [list(map(int, r)) for r in np.asarray(ids)]
        return self._step_all()

    def PrefillRagged(self, prompts, opts):
        self.calls.append(("ragged", [len(p) for p in prompts]))
        self.seqs = [list(map(int, p)) for p in prompts]
        return self._step_all()

    def _step_all(self):
        out = []
        for s in self.seqs:
            t = 0 if (len(s) > 1 and s[-1] == 0) else self._next(s[-1])   # an ended sequence stands still
            s.append(t)
            out.append(t)
        return np.asarray(out, dtype=np.int32)

    def Decode(self, n, opts, stop_on_eos=False):
        cols = []
        for _ in range(n):
            cols.append(self._step_all())
            if stop_on_eos and all(s[-1] == 0 for s in self.seqs):
                break
        return np.stack(cols, axis=1)


def _vocab12():
    return Vocab(["w%d" % i for i in range(5, 12)])     # ids 5..11 = w5..w11, 12 entries: no pad


def test_runner_file_to_file(tmp_path):
    vocab = _vocab12()
    src = tmp_path / "in.txt"
    src.write_text("w5\nw9 w10\nw6 w5 w6\n", encoding="utf-8")
    dst = tmp_path / "out.txt"
    eng = _EchoEngine()
    opts = DecodingOptions(MaxSrcSentLength=16, MaxTgtSentLength=8)
    run = GptTextRunner(eng, vocab, opts)
    lines = run.Test(str(src), str(dst), batch_size=2)
    # line 0: <s> w5 -> w6 w7 </s>; line 1: <s> w9 w10 -> w11 then id 0 (12 mod 12) = </s>; line 2 (batch of its own):
    # <s> w6 w5 w6 -> w7 </s>
    assert lines == ["<s> w5 w6 w7 </s>", "<s> w9 w10 w11 </s>", "<s> w6 w5 w6 w7 </s>"]
    assert dst.read_text(encoding="utf-8").splitlines() == lines
    assert eng.calls[0] == ("ragged", [2, 3]) and eng.calls[1] == ("prefill", (1, 4))
    assert run.stats.lines == 3 and run.stats.prompt_tokens == 9 and run.stats.new_tokens == 3 + 2 + 2


def test_runner_respects_max_target_length(tmp_path):
    vocab = _vocab12()
    eng = _EchoEngine(V=400)                # never reaches </s> through the modulus
    opts = DecodingOptions(MaxSrcSentLength=16, MaxTgtSentLength=6)
    run = GptTextRunner(eng, vocab, opts)
    out = run.run_batch([["<s>", "w8"], ["<s>", "w8", "w9", "w10"]])[0]
    # every line ends at MaxTgtSentLength tokens in total (the loop `for i = promptLen; i < MaxTgtSentLength`)
    assert [len(o) for o in out] == [6, 6]
    assert out[0][:3] == ["<s>", "w8", "w9"] and out[1][4:] == ["w11", "<unk>"]
    # a prompt that already fills the limit gets nothing
    out = GptTextRunner(eng, vocab, DecodingOptions(MaxTgtSentLength=2)).run_batch([["<s>", "w8"]])[0]
    assert out == [["<s>", "w8"]]


def test_runner_writes_all_beams_of_a_line(tmp_path):
    from tests.test_beam_cpu import _FakeEngine, _TableModel
    vocab = Vocab(["w%d" % i for i in range(5, 23)] + ["x"])          # 24 entries
    model = _TableModel(V=24, seed=5, eos_boost=0.5)
    eng = _FakeEngine(model, max_batch=4)                              # room for two lines of two beams
    opts = DecodingOptions(MaxSrcSentLength=16, MaxTgtSentLength=9, BeamSearchSize=2)
    src = tmp_path / "in.txt"
    src.write_text("w5 w6\nw7 w8\nw9\n", encoding="utf-8")
    run = GptTextRunner(eng, vocab, opts)
    lines = run.Test(str(src), None, batch_size=3)
    assert len(lines) == 3
    from seq2seqsharp_b200.beam import beam_search
    for text, line in zip(["w5 w6", "w7 w8", "w9"], lines):
        beams = line.split("\t")
        assert len(beams) == 2
        words = ["<s>"] + text.split(" ")
        alone = beam_search(_FakeEngine(model, max_batch=2), [vocab.GetWordIndex([words])[0]], opts)
        for k, beam in enumerate(beams):
            want = words + vocab.ConvertIdsToString(alone.ids[k][0])
            if "</s>" in want:
                want = want[: want.index("</s>") + 1]
            assert beam.split(" ") == want
