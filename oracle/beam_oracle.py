"""TEST INFRASTRUCTURE: CPU restatement of the reference's beam search around the GPT decoder.  Only tests may import it.

Follows, statement by statement:
  * the fixed-size two-heap queue                      AdvUtils/FixedSizePriorityQueue.cs:15-314
  * its comparer (descending: smaller score first)      Seq2SeqSharp/Tools/ComparableItem.cs:29-48, Utils/BeamSearch.cs:36-46
  * the candidate loop of a decode step                  Seq2SeqSharp/Applications/Decoder.cs:447-517 (same loop in GPTDecode)
  * the loop over steps, beams and batch items           Seq2SeqSharp/Applications/GPT.cs:236-310
As the reference does with more than one beam, every hypothesis is run from its first token at every step (no KV cache).
Parity unpinned: no reference-held output exists for this path (no dotnet here); the restatement is checked against
hand-worked queue cases in tests/test_beam_cpu.py.
"""
import numpy as np


class FixedSizePriorityQueue:
    def __init__(self, capacity, compare):
        if capacity < 1:
            raise Exception("priority queue capacity must be at least one!")
        self.m_iCount = 0
        self.m_iCapacity = capacity
        self.m_iBottomSize = self.m_iTopSize = 0
        iBottomCapacity = max(capacity // 2, 1)
        iTopCapacity = max(capacity - iBottomCapacity, 1)
        self.m_rgtTop = [None] * iTopCapacity
        self.m_rgtBottom = [None] * iBottomCapacity
        self.compare = compare

    def Enqueue(self, t):
        if self.m_iCapacity == self.m_iCount:
            if self.m_iCapacity == 1:
                if not self.Better(t, self.m_rgtTop[0], True):
                    return False
                self.m_rgtTop[0] = t
                return True
            if not self.Better(t, self.m_rgtBottom[0], True):
                return False
            self.m_rgtBottom[0] = t
            iUpdated = self.DownHeapify(self.m_rgtBottom, 0, self.m_iBottomSize, False)
            if not self.SemiLeaf(iUpdated, self.m_iBottomSize):
                return True
            iTop = self.CheckBoundaryUpwards(iUpdated)
            if iTop == -1:
                return True
            self.UpHeapify(self.m_rgtTop, iTop, self.m_iTopSize, True)
            return True
        self.m_iCount += 1
        if self.m_iBottomSize < self.m_iTopSize:
            iPos = self.m_iBottomSize
            self.m_iBottomSize += 1
            self.m_rgtBottom[iPos] = t
            iUp = self.CheckBoundaryUpwards(iPos)
            if iUp == -1:
                self.UpHeapify(self.m_rgtBottom, iPos, self.m_iBottomSize, False)
            else:
                self.UpHeapify(self.m_rgtTop, iUp, self.m_iTopSize, True)
            return True
        iPos = self.m_iTopSize
        self.m_iTopSize += 1
        self.m_rgtTop[iPos] = t
        iBottom = self.CheckBoundaryDownwards(iPos)
        if iBottom == -1:
            self.UpHeapify(self.m_rgtTop, iPos, self.m_iTopSize, True)
        else:
            self.UpHeapify(self.m_rgtBottom, iBottom, self.m_iBottomSize, False)
        return True

    @staticmethod
    def Parent(i):
        return (i - 1) // 2 if i > 0 else 0      # C# (0 - 1) / 2 == 0

    @staticmethod
    def Left(i):
        return 2 * i + 1

    @staticmethod
    def Right(i):
        return 2 * i + 2

    def SemiLeaf(self, i, iSize):
        return self.Right(i) >= iSize

    def BottomNode(self, i):
        if i < self.m_iBottomSize:
            return i
        if i % 2 == 1:
            return self.Parent(i)
        return i - 1

    def TopNode1(self, i):
        if self.Left(i) >= self.m_iBottomSize and self.Left(i) < self.m_iTopSize:
            return self.Left(i)
        return i

    def TopNode2(self, i):
        if i == self.m_iBottomSize - 1 and 1 == (i % 2) and self.m_iTopSize > self.m_iBottomSize:
            return i + 1
        if self.Left(i) >= self.m_iBottomSize and self.Left(i) < self.m_iTopSize:
            return self.Left(i)
        return i

    def UpHeapify(self, rgt, i, iSize, fTop):
        while i > 0:
            iPar = self.Parent(i)
            if not self.Better(rgt[i], rgt[iPar], fTop):
                return i
            rgt[i], rgt[iPar] = rgt[iPar], rgt[i]
            i = iPar
        return i

    def DownHeapify(self, rgt, i, iSize, fTop):
        while True:
            iLeft, iRight = self.Left(i), self.Right(i)
            iLargest = i
            if iLeft < iSize and self.Better(rgt[iLeft], rgt[iLargest], fTop):
                iLargest = iLeft
            if iRight < iSize and self.Better(rgt[iRight], rgt[iLargest], fTop):
                iLargest = iRight
            if iLargest == i:
                return i
            rgt[i], rgt[iLargest] = rgt[iLargest], rgt[i]
            i = iLargest

    def CheckBoundaryUpwards(self, iBottomPos):
        iTop1 = self.TopNode1(iBottomPos)
        iTop2 = self.TopNode2(iBottomPos)
        iBetter = -1
        if self.Better(self.m_rgtBottom[iBottomPos], self.m_rgtTop[iTop1], True):
            iBetter = iTop1
        if self.Better(self.m_rgtBottom[iBottomPos], self.m_rgtTop[iTop2], True) and \
                (iBetter == -1 or self.Better(self.m_rgtTop[iTop1], self.m_rgtTop[iTop2], True)):
            iBetter = iTop2
        if iBetter == -1:
            return -1
        self.m_rgtTop[iBetter], self.m_rgtBottom[iBottomPos] = self.m_rgtBottom[iBottomPos], self.m_rgtTop[iBetter]
        return iBetter

    def CheckBoundaryDownwards(self, iTopPos):
        iBottomPos = self.BottomNode(iTopPos)
        if iBottomPos == -1:
            return -1
        if iBottomPos >= self.m_iBottomSize or not self.Better(self.m_rgtBottom[iBottomPos], self.m_rgtTop[iTopPos], True):
            return -1
        self.m_rgtTop[iTopPos], self.m_rgtBottom[iBottomPos] = self.m_rgtBottom[iBottomPos], self.m_rgtTop[iTopPos]
        return iBottomPos

    def Better(self, t1, t2, fTop):
        i = self.compare(t1, t2)
        return i > 0 if fTop else i < 0

    def __iter__(self):
        for i in range(self.m_iTopSize):
            yield self.m_rgtTop[i]
        for i in range(self.m_iBottomSize - 1, -1, -1):
            yield self.m_rgtBottom[i]


def _compare_descending(x, y):
    """ComparableItemComparer(false): sign of (x.Score - y.Score), negated."""
    d = np.float32(x[0]) - np.float32(y[0])
    return -int(np.sign(d))


def GetTopNBSS(bssList, topN):
    """Utils/BeamSearch.cs:36-46; bssList items are (Score, OutputIds)."""
    q = FixedSizePriorityQueue(topN, _compare_descending)
    for bss in bssList:
        q.Enqueue(bss)
    return list(q)


def candidates(probs, beam_size):
    """Decoder.cs:459-517: beam_size rounds of ArgMax (first maximum), Gather + Log, ScatterFill 0 on a copy of probs [B, V]."""
    p = np.array(probs, dtype=np.float32, copy=True)
    out = []
    for _ in range(beam_size):
        idx = np.argmax(p, axis=1)                       # numpy's first-maximum rule = the reference's ArgMax
        val = p[np.arange(p.shape[0]), idx]
        out.append((idx.astype(np.int64), np.log(val.astype(np.float32)).astype(np.float32)))
        p[np.arange(p.shape[0]), idx] = 0.0
    return out


def beam_search(oracle_gpt, prompts, opts, record=None):
    """GPT.cs:236-310 for BeamSearchSize >= 1, greedy.  Returns ([beam][batch] generated ids, [beam][batch] scores).
    `record(step, batch2beam2seq)` sees the kept hypotheses (Score, OutputIds) of every step."""
    prompts = np.asarray(prompts, dtype=np.int32)
    batchSize, promptLen = prompts.shape
    beamSize = int(opts.BeamSearchSize)
    blocked = opts.BlockedTokens or ()
    # InitBeamSearchStatusListList: one beam, Score = 1.0f
    beam2batchStatus = [[(np.float32(1.0), [int(t) for t in prompts[b]]) for b in range(batchSize)]]
    for i in range(promptLen, int(opts.MaxTgtSentLength)):
        batch2beam2seq = None
        for batchStatus in beam2batchStatus:
            tokens = np.asarray([s[1] for s in batchStatus], dtype=np.int32)
            oracle_gpt.reset()
            _, probs = oracle_gpt.step(tokens, 1.0, blocked)     # whole texts, no cache: last position's probabilities
            bssSeqList = []
            for idx, logp in candidates(probs, beamSize):
                bssSeqList.append([(np.float32(batchStatus[b][0] + np.float32(-1.0) * logp[b]) if beamSize > 1 else np.float32(1.0),
                                    batchStatus[b][1] + [int(idx[b])]) for b in range(batchSize)])
            swapped = [[bssSeqList[k][b] for k in range(beamSize)] for b in range(batchSize)]
            batch2beam2seq = swapped if batch2beam2seq is None else [batch2beam2seq[b] + swapped[b] for b in range(batchSize)]
        if beamSize > 1:
            batch2beam2seq = [GetTopNBSS(batch2beam2seq[b], beamSize) for b in range(batchSize)]
        if record is not None:
            record(i - promptLen, batch2beam2seq)
        beam2batchStatus = [[batch2beam2seq[b][k] for b in range(batchSize)] for k in range(len(batch2beam2seq[0]))]
        if all(s[1][-1] == 0 for bs in beam2batchStatus for s in bs):
            break
    ids = [[s[1][promptLen:] for s in bs] for bs in beam2batchStatus]
    scores = [[float(s[0]) for s in bs] for bs in beam2batchStatus]
    return ids, scores
