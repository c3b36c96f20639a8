"""Text in, text out around the GPT token loop: vocabulary, SentencePiece, the line reader and the line writer.

Host-side mirror of what the reference's test mode does around `GPT.RunForwardOnSingleDevice`
(Tools/BaseSeq2SeqFramework.cs:987-992 `Test<X>`, :1001-1045 `RunTest`):

  input file --SntBatchStreamReader--> token lists --Vocab--> ids --token loop--> ids --Vocab--> words
             --CombineInputOutput / RemoveDuplicatedEOS--> lines --SntBatchStreamWriter (+ SentencePiece)--> output file

Nothing here touches the GPU; the engine is whatever object is handed to `GptTextRunner` (`seq2seqsharp_b200.gpt.GPT`).
"""
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np


class BuildInTokens:
    """Corpus/BuildInTokens.cs:17-27."""
    EOS = "</s>"
    BOS = "<s>"
    UNK = "<unk>"
    SEP = "[SEP]"
    CLS = "[CLS]"

    @staticmethod
    def IsPreDefinedToken(s: str) -> bool:
        return s in (BuildInTokens.EOS, BuildInTokens.BOS, BuildInTokens.UNK, BuildInTokens.CLS, BuildInTokens.SEP)


class SENTTAGS:
    """Utils/Vocab.cs:20-27: the ids of the built-in tokens."""
    END, START, UNK, SEP, CLS = range(5)


class Vocab:
    """Token <-> id table (Utils/Vocab.cs:30-346).  Ids 0..4 are </s>, <s>, <unk>, [SEP], [CLS]; the words of a
    vocabulary file follow in file order (first tab-separated column, built-in tokens skipped); a table with an odd number
    of entries gets `[PAD_0]` appended (Vocab.cs:118-146).  Unknown words map to <unk>, unknown ids print as <unk>."""

    def __init__(self, words: Optional[Sequence[str]] = None, ignore_case: bool = False):
        self.IgnoreCase = bool(ignore_case)
        self.Items: List[str] = [BuildInTokens.EOS, BuildInTokens.BOS, BuildInTokens.UNK, BuildInTokens.SEP, BuildInTokens.CLS]
        self.WordToIndex: Dict[str, int] = {w: i for i, w in enumerate(self.Items)}
        self.IndexToWord: Dict[int, str] = {i: w for i, w in enumerate(self.Items)}
        if words is not None:
            for w in words:
                self._add(w)
            self._align()

    def _key(self, w: str) -> str:
        return w.lower() if self.IgnoreCase else w

    def _add(self, word: str):
        if BuildInTokens.IsPreDefinedToken(word):
            return
        q = len(self.IndexToWord)
        self.Items.append(word)
        self.WordToIndex[self._key(word)] = q
        self.IndexToWord[q] = word

    def _align(self):
        if len(self.IndexToWord) % 2 != 0:
            self._add("[PAD_0]")

    @classmethod
    def from_file(cls, path: str) -> "Vocab":
        """`Vocab(string vocabFilePath)`: one word per line, anything after the first tab ignored."""
        with open(path, encoding="utf-8") as fh:
            lines = fh.read().splitlines()
        return cls([ln.split("\t")[0] for ln in lines])

    @classmethod
    def from_index_table(cls, index_to_word: Sequence[str], ignore_case: bool = False) -> "Vocab":
        """The table a model file stores (`Vocab(Vocab_4_ProtoBufSerializer)`, Vocab.cs:49-60): taken as it is, position =
        id, nothing skipped or appended."""
        v = cls.__new__(cls)
        v.IgnoreCase = bool(ignore_case)
        v.Items = list(index_to_word)
        v.IndexToWord = {i: w for i, w in enumerate(index_to_word)}
        v.WordToIndex = {}
        for i, w in enumerate(index_to_word):
            v.WordToIndex[v._key(w)] = i
        return v

    @property
    def Count(self) -> int:
        return len(self.IndexToWord)

    def DumpVocab(self, path: str):
        """Vocab.cs:155-164: `word<TAB>id` per line."""
        with open(path, "w", encoding="utf-8") as fh:
            for i, w in self.IndexToWord.items():
                fh.write("%s\t%d\n" % (w, i))

    def GetString(self, idx: int) -> str:
        return self.IndexToWord.get(int(idx), BuildInTokens.UNK)

    def GetWordIndex(self, word_or_seqs):
        """One word -> id, or a list of token lists -> a list of id lists (Vocab.cs:296-344)."""
        if isinstance(word_or_seqs, str):
            return self.WordToIndex.get(self._key(word_or_seqs), SENTTAGS.UNK)
        return [[self.WordToIndex.get(self._key(w), SENTTAGS.UNK) for w in seq] for seq in word_or_seqs]

    def ConvertIdsToString(self, ids):
        """A list of ids -> words, or a list of id lists -> a list of word lists (Vocab.cs:181-252)."""
        ids = list(ids)
        if ids and isinstance(ids[0], (list, tuple, np.ndarray)):
            return [[self.GetString(i) for i in seq] for seq in ids]
        return [self.GetString(i) for i in ids]


class SentencePiece:
    """The reference binds the SentencePiece C++ library (`_SentencePiece/SentencePiece.cs:185-275`): `Encode(text)` gives
    the pieces joined by blanks, `Decode(pieces joined by blanks)` the text, trimmed.  Here the same library is reached
    through its Python package (an image without it gets an ImportError at construction, not a silent pass-through)."""

    def __init__(self, model_path: str):
        import sentencepiece as spm
        self._sp = spm.SentencePieceProcessor(model_file=model_path)

    def Encode(self, text: str, toLower: bool = False) -> str:
        if toLower:
            text = text.lower()
        return " ".join(self._sp.encode(text, out_type=str))

    def Decode(self, pieces) -> str:
        if not isinstance(pieces, str):
            pieces = " ".join(pieces)
        return self._sp.decode_pieces(pieces.split(" ")).strip()


def AppendNewBatch(batch: List[List[str]], line: str, max_token_length: int):
    """Utils/Misc.cs:83-91: trim, split at single blanks, keep at most max - 2 tokens (room for <s> and </s>)."""
    tokens = line.strip().split(" ")
    if len(tokens) > max_token_length - 2:
        tokens = tokens[: max(0, max_token_length - 2)]
    batch.append(tokens)


def TryAddPrefix(token_lists: List[List[str]], prefix: str):
    """Corpus/CorpusBatch.cs:35-51."""
    for t in token_lists:
        if not t or t[0] != prefix:
            t.insert(0, prefix)


class SntBatchStreamReader:
    """Corpus/SntBatchStreamReader.cs:20-75 with the batch type the GPT console uses (`SeqCorpusBatch.CreateBatch(src,
    null)`, Corpus/SeqCorpusBatch.cs:29-47: every line gets <s> in front, no </s> behind).  `GetNextBatch()` returns
    (index of the batch's first line, token lists) or (-1, None) at the end of the file."""

    def __init__(self, file_path: str, batch_size: int, max_sent_length: int, sentence_piece: Optional[SentencePiece] = None):
        self._fh = open(file_path, encoding="utf-8")
        self._idx = 0
        self.batch_size, self.max_sent_length, self.sp = int(batch_size), int(max_sent_length), sentence_piece

    def GetNextBatch(self) -> Tuple[int, Optional[List[List[str]]]]:
        batch: List[List[str]] = []
        first = self._idx
        while len(batch) < self.batch_size:
            line = self._fh.readline()
            if line == "":
                break
            line = line.rstrip("\r\n")
            if self.sp is not None:
                line = self.sp.Encode(line)
            AppendNewBatch(batch, line, self.max_sent_length)
            self._idx += 1
        if not batch:
            return -1, None
        TryAddPrefix(batch, BuildInTokens.BOS)
        return first, batch

    def close(self):
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def RemoveDuplicatedEOS(sentences: List[List[str]]):
    """Tools/BaseSeq2SeqFramework.cs:73-87: everything after a sentence's first </s> goes, one </s> stays."""
    for snt in sentences:
        if BuildInTokens.EOS in snt:
            del snt[snt.index(BuildInTokens.EOS) + 1:]


class SntBatchStreamWriter:
    """Corpus/SntBatchStreamWriter.cs:16-227 without the alignment file: batches may arrive in any order, lines leave in
    input order (a line is written once every line before it has been), the beams of a line are joined by tabs, and a
    SentencePiece model, if given, turns the line of pieces back into text."""

    def __init__(self, file_path: Optional[str] = None, sentence_piece: Optional[SentencePiece] = None):
        self._fh = open(file_path, "w", encoding="utf-8") if file_path else None
        self.sp = sentence_piece
        self._buffer: List[Optional[str]] = []
        self._written = 0
        self.lines: List[str] = []      # what has been written, also kept when there is no file

    def WriteResults(self, idx: int, output: List[List[List[str]]]):
        """output[beam][sequence] = words of line idx + sequence."""
        n = len(output[0])
        finals = ["\t".join(" ".join(output[beam][b]) for beam in range(len(output))) for b in range(n)]
        while len(self._buffer) < idx + n - self._written:
            self._buffer.append(None)
        for i, line in enumerate(finals):
            self._buffer[idx + i - self._written] = line
        end = 0
        while end < len(self._buffer) and self._buffer[end] is not None:
            line = self._buffer[end]
            if self.sp is not None:
                line = self.sp.Decode(line)
            self.lines.append(line)
            if self._fh:
                self._fh.write(line + "\n")
            end += 1
        if end:
            del self._buffer[:end]
            self._written += end

    def Close(self):
        if self._fh:
            self._fh.close()
            self._fh = None


@dataclass
class TextStats:
    lines: int = 0
    prompt_tokens: int = 0
    new_tokens: int = 0


class GptTextRunner:
    """`GPT.Test(inputFile, outputFile, batchSize, decodingOptions, srcSpm, tgtSpm)` for this engine.

    Per batch of lines: words -> ids (`TgtVocab.GetWordIndex`, GPT.cs:219), the token loop until every sequence has ended or
    reached `MaxTgtSentLength`, ids -> words, prompt + generated words per line (`CombineInputOutput`, GPT.cs:182-200),
    `RemoveDuplicatedEOS`, writer.

    The reference pads the prompts of a batch to one length with </s> and decodes all of them from that length
    (Decoder.cs:656); a shorter line of a batch is therefore continued after padding it never asked for.  Here every line is
    continued from its own end (`PrefillRagged` / the slot scheduler), which is what the reference produces for that line in
    a batch of its own; for batches of equally long lines the two agree."""

    def __init__(self, gpt, vocab: Vocab, opts, use_scheduler: bool = False, slots: Optional[int] = None):
        self.gpt, self.vocab, self.opts = gpt, vocab, opts
        self.use_scheduler, self.slots = bool(use_scheduler), slots
        self.stats = TextStats()

    def _generate(self, prompts: List[List[int]]) -> List[List[int]]:
        """ids generated for each prompt (a final 0 = </s> kept), at most MaxTgtSentLength - len(prompt) of them."""
        max_len = int(self.opts.MaxTgtSentLength)
        lens = [len(p) for p in prompts]
        # one batch runs until its shortest line has reached the limit; the longest line then holds max - min tokens more
        # than it may print (cut below).  Where the engine's cache has no room for that, the slots take the lines one by
        # one, each with its own budget.
        cap = getattr(self.gpt, "max_tokens", None)
        crowded = cap is not None and max_len + (max(lens) - min(lens)) > int(cap)
        if self.use_scheduler or crowded:
            from .scheduler import ContinuousBatcher, Request
            reqs = [Request(i, p, max_len - len(p)) for i, p in enumerate(prompts)]
            out = ContinuousBatcher(self.gpt, self.opts, self.slots or len(prompts), max_tokens=max_len).run(reqs)
            return [[int(t) for t in out[i]] for i in range(len(prompts))]
        n_new = max_len - min(lens)
        if n_new <= 0:
            return [[] for _ in prompts]
        self.gpt.Reset()
        if len(set(lens)) == 1:
            first = self.gpt.Prefill(np.asarray(prompts, dtype=np.int32), self.opts)
        else:
            first = self.gpt.PrefillRagged(prompts, self.opts)
        gen = [[int(t)] for t in first]
        steps = n_new - 1
        if steps > 0 and any(g[0] != 0 for g in gen):
            ids = self.gpt.Decode(steps, self.opts, stop_on_eos=True)
            for b in range(len(prompts)):
                gen[b].extend(int(t) for t in ids[b])
        out = []
        for b, g in enumerate(gen):
            g = g[: max(0, max_len - lens[b])]
            if 0 in g:
                g = g[: g.index(0) + 1]
            out.append(g)
        return out

    def _run_beams(self, token_lists: List[List[str]], prompts: List[List[int]]) -> List[List[List[str]]]:
        """BeamSearchSize > 1: output[beam][sequence], beams in the reference's order.  Lines of one length share a search
        while the engine has sequences for all their hypotheses; otherwise the lines are searched one after the other."""
        from .beam import beam_search
        K = int(self.opts.BeamSearchSize)
        out = [[None] * len(prompts) for _ in range(K)]
        groups: Dict[int, List[int]] = {}
        for i, p in enumerate(prompts):
            groups.setdefault(len(p), []).append(i)
        per_call = max(1, int(getattr(self.gpt, "max_batch", K)) // K)
        for idxs in groups.values():
            for at in range(0, len(idxs), per_call):
                part = idxs[at:at + per_call]
                res = beam_search(self.gpt, np.asarray([prompts[i] for i in part], dtype=np.int32), self.opts)
                for k in range(K):
                    for j, i in enumerate(part):
                        gen = res.ids[k][j] if k < len(res.ids) else []
                        out[k][i] = list(token_lists[i]) + self.vocab.ConvertIdsToString(list(gen))
                        self.stats.new_tokens += len(gen)
        for beam in out:
            RemoveDuplicatedEOS(beam)
        self.stats.lines += len(token_lists)
        self.stats.prompt_tokens += sum(len(p) for p in prompts)
        return out

    def run_batch(self, token_lists: List[List[str]]) -> List[List[List[str]]]:
        """token lists (with <s>) -> output[beam][sequence] = prompt words + generated words (one beam unless
        BeamSearchSize > 1)."""
        prompts = self.vocab.GetWordIndex(token_lists)
        if int(getattr(self.opts, "BeamSearchSize", 1)) > 1:
            return self._run_beams(token_lists, prompts)
        gen = self._generate(prompts)
        words = self.vocab.ConvertIdsToString([list(g) for g in gen]) if gen else []
        combined = [list(t) + list(w) for t, w in zip(token_lists, words)]
        RemoveDuplicatedEOS(combined)
        self.stats.lines += len(token_lists)
        self.stats.prompt_tokens += sum(len(p) for p in prompts)
        self.stats.new_tokens += sum(len(g) for g in gen)
        return [combined]

    def Test(self, input_file: str, output_file: Optional[str], batch_size: int, src_spm_path: Optional[str] = None,
             tgt_spm_path: Optional[str] = None) -> List[str]:
        src_sp = SentencePiece(src_spm_path) if src_spm_path else None
        tgt_sp = SentencePiece(tgt_spm_path) if tgt_spm_path else None
        writer = SntBatchStreamWriter(output_file, tgt_sp)
        with SntBatchStreamReader(input_file, batch_size, int(self.opts.MaxSrcSentLength), src_sp) as reader:
            while True:
                idx, batch = reader.GetNextBatch()
                if idx < 0:
                    break
                writer.WriteResults(idx, self.run_batch(batch))
        writer.Close()
        return writer.lines
