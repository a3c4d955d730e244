"""Word2Vec, ParagraphVectors and their vocabulary / Huffman machinery.

Parity: ``deeplearning4j-nlp/.../models/word2vec/Word2Vec.java``, ``models/paragraphvectors/ParagraphVectors.java``,
``models/sequencevectors/SequenceVectors.java``, ``models/embeddings/learning/impl/elements/{SkipGram,CBOW}.java``,
``models/embeddings/learning/impl/sequence/{DBOW,DM}.java``, ``models/word2vec/Huffman.java`` and the native
``skipgram`` / ``cbow`` ops (``libnd4j/include/ops/declarable/generic/nlp``).

The reference trains one (word, context) pair at a time from several CPU threads.  Here an epoch's training
pairs are generated as tensors on the device (dynamic windows, frequent-word subsampling, sentence boundaries
respected), shuffled and consumed in large batches: gathers of the embedding rows, one fused sigmoid / gradient
expression, and ``index_add_`` scatter updates.  Negative sampling draws from the unigram^0.75 table with
``torch.multinomial``; hierarchical softmax uses padded Huffman code / point matrices.
"""
from __future__ import annotations

import heapq
import json
import math
import struct
import zipfile

import numpy as np
import torch

from ..nd.ndarray import INDArray
from .tokenization import (CollectionSentenceIterator, DefaultTokenizerFactory, LabelledDocument, LabelsSource, SentenceIterator,
                           SentenceIteratorConverter)


# ----------------------------------------------------------------------------- vocabulary
class VocabWord:
    __slots__ = ("word", "count", "index", "codes", "points", "is_label")

    def __init__(self, word, count=1.0, index=-1, is_label=False):
        self.word, self.count, self.index, self.codes, self.points, self.is_label = word, float(count), index, [], [], is_label

    def getWord(self): return self.word
    getLabel = getWord
    def getElementFrequency(self): return self.count
    def getIndex(self): return self.index
    def getCodes(self): return self.codes
    def getPoints(self): return self.points
    def isLabel(self): return self.is_label


class VocabCache:
    """``AbstractCache``: word <-> index, frequencies, total counts."""

    def __init__(self):
        self.words, self.by_index, self.total = {}, [], 0.0

    def addToken(self, vw):
        self.words[vw.word] = vw
    def incrementWordCount(self, w, by=1):
        vw = self.words.get(w)
        if vw is None:
            vw = self.words[w] = VocabWord(w, 0)
        vw.count += by
        self.total += by
    def finalize_(self, minFrequency=1, keep=()):
        kept = [v for v in self.words.values() if v.count >= minFrequency or v.word in keep or v.is_label]
        kept.sort(key=lambda v: (-v.count, v.word))
        self.words = {v.word: v for v in kept}
        self.by_index = kept
        for i, v in enumerate(kept):
            v.index = i
    def containsWord(self, w): return w in self.words
    hasToken = containsWord
    def wordFor(self, w): return self.words.get(w)
    tokenFor = wordFor
    def indexOf(self, w): return self.words[w].index if w in self.words else -1
    def wordAtIndex(self, i): return self.by_index[i].word if 0 <= i < len(self.by_index) else None
    def elementAtIndex(self, i): return self.by_index[i]
    def wordFrequency(self, w): return int(self.words[w].count) if w in self.words else 0
    def numWords(self): return len(self.by_index)
    def words_(self): return [v.word for v in self.by_index]
    def vocabWords(self): return list(self.by_index)
    def totalWordOccurrences(self): return self.total


def build_huffman(vocab: VocabCache):
    """Binary Huffman tree over word frequencies: fills ``codes`` / ``points`` of every word (``Huffman.java``)."""
    n = vocab.numWords()
    if n < 2:
        for v in vocab.by_index:
            v.codes, v.points = [0], [0]
        return 1
    heap = [(v.count, i, i) for i, v in enumerate(vocab.by_index)]
    heapq.heapify(heap)
    parent, binary = {}, {}
    nxt = n
    while len(heap) > 1:
        c1, _, a = heapq.heappop(heap)
        c2, _, b = heapq.heappop(heap)
        parent[a], parent[b] = nxt, nxt
        binary[a], binary[b] = 0, 1
        heapq.heappush(heap, (c1 + c2, nxt, nxt))
        nxt += 1
    root = nxt - 1
    for i, v in enumerate(vocab.by_index):
        codes, points, node = [], [], i
        while node != root:
            codes.append(binary[node])
            node = parent[node]
            points.append(node - n)
        v.codes, v.points = codes[::-1], points[::-1]
    return n - 1                                                      # number of inner nodes


# ----------------------------------------------------------------------------- lookup table
class InMemoryLookupTable:
    def __init__(self, vocab, layerSize, seed=42, device="cpu", useHS=False, negative=0, inner_nodes=0):
        self.vocab, self.layerSize = vocab, layerSize
        g = torch.Generator().manual_seed(int(seed))
        n = vocab.numWords()
        self.syn0 = ((torch.rand(n, layerSize, generator=g) - 0.5) / layerSize).to(device)
        self.syn1 = torch.zeros(max(inner_nodes, 1), layerSize, device=device) if useHS else None
        self.syn1Neg = torch.zeros(n, layerSize, device=device) if negative > 0 else None

    def getSyn0(self): return INDArray(self.syn0)
    def getSyn1(self): return None if self.syn1 is None else INDArray(self.syn1)
    def getSyn1Neg(self): return None if self.syn1Neg is None else INDArray(self.syn1Neg)
    def vector(self, w):
        i = self.vocab.indexOf(w)
        return None if i < 0 else INDArray(self.syn0[i])
    def layerSize_(self): return self.layerSize
    def getVocabCache(self): return self.vocab


def _scatter_add(table, idx, upd, cap=8.0):
    """``table[idx] += upd`` with duplicate control: a row hit more than ``cap`` times in one batch receives ``cap`` times
    the mean of its updates instead of their sum.  Up to ``cap`` duplicates this equals sequential (hogwild) updates with
    stale values; beyond it the step stays bounded, which matters for very frequent words and tiny vocabularies."""
    cnt = torch.bincount(idx, minlength=table.shape[0]).to(upd.dtype)[idx]
    table.index_add_(0, idx, upd * (cap / cnt.clamp(min=cap)).unsqueeze(1))


# ----------------------------------------------------------------------------- SequenceVectors base
class SequenceVectors:
    def __init__(self, **kw):
        d = dict(minWordFrequency=5, iterations=1, epochs=1, layerSize=100, seed=42, windowSize=5, learningRate=0.025,
                 minLearningRate=1e-4, negativeSample=0, useHierarchicSoftmax=True, sampling=0.0, batchSize=2048,
                 elementsLearningAlgorithm="SkipGram", sequenceLearningAlgorithm="DBOW", tokenizerFactory=None, iterate=None,
                 stopWords=(), trainElementsRepresentation=True, trainSequencesRepresentation=True, device=None, labelsSource=None,
                 useUnknown=False, unknownElement="UNK", workers=1, useAdaGrad=False, vocabCache=None, lookupTable=None,
                 allowParallelTokenization=False, modelUtils=None, limitVocabularySize=0)
        for k, v in kw.items():
            if k not in d:
                raise TypeError(f"unknown option {k}")
        d.update(kw)
        self.__dict__.update(d)
        algo = self.elementsLearningAlgorithm
        self.elementsLearningAlgorithm = algo if isinstance(algo, str) else type(algo).__name__
        sa = self.sequenceLearningAlgorithm
        self.sequenceLearningAlgorithm = sa if isinstance(sa, str) else type(sa).__name__
        self.tokenizerFactory = self.tokenizerFactory or DefaultTokenizerFactory()
        self.device = torch.device(self.device) if self.device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.vocab = self.vocabCache
        self.lookupTable = self.lookupTable
        if self.useHierarchicSoftmax is False and self.negativeSample <= 0:
            self.negativeSample = 5

    # -- corpus
    def _sequences(self):
        """Yields (tokens, labels) per sequence."""
        it = self.iterate
        if it is None:
            raise ValueError("no corpus: set iterate(...)")
        if isinstance(it, (list, tuple)) and (not it or isinstance(it[0], str)):
            it = CollectionSentenceIterator(it)
        stop = set(self.stopWords or ())
        if isinstance(it, SentenceIterator):
            for s in it:
                yield [t for t in self.tokenizerFactory.create(s).getTokens() if t not in stop], []
        else:
            for d in it:
                yield [t for t in self.tokenizerFactory.create(d.getContent()).getTokens() if t not in stop], list(d.getLabels())

    def buildVocab(self):
        vocab = VocabCache()
        labels = []
        for toks, labs in self._sequences():
            for t in toks:
                vocab.incrementWordCount(t)
            for l in labs:
                if l not in vocab.words:
                    vocab.addToken(VocabWord(l, 1.0, is_label=True))
                    labels.append(l)
        if self.useUnknown:
            vocab.addToken(VocabWord(self.unknownElement, 1.0))
        vocab.finalize_(self.minWordFrequency, keep=(self.unknownElement,) if self.useUnknown else ())
        if self.limitVocabularySize and vocab.numWords() > self.limitVocabularySize:
            keep = {v.word for v in vocab.by_index[:self.limitVocabularySize]} | set(labels)
            vocab.words = {w: v for w, v in vocab.words.items() if w in keep}
            vocab.finalize_(0)
        self.vocab = vocab
        inner = build_huffman(vocab) if self.useHierarchicSoftmax else 0
        self.lookupTable = InMemoryLookupTable(vocab, self.layerSize, self.seed, self.device, self.useHierarchicSoftmax, self.negativeSample, inner)
        return self

    def _corpus_tensors(self):
        ids, sent, doc_ids = [], [], []
        unk = self.vocab.indexOf(self.unknownElement) if self.useUnknown else -1
        for s, (toks, labs) in enumerate(self._sequences()):
            idx = [self.vocab.indexOf(t) for t in toks]
            idx = [i if i >= 0 else unk for i in idx]
            idx = [i for i in idx if i >= 0]
            ids.extend(idx)
            sent.extend([s] * len(idx))
            doc_ids.append([self.vocab.indexOf(l) for l in labs])
        return (torch.tensor(ids, dtype=torch.long, device=self.device), torch.tensor(sent, dtype=torch.long, device=self.device), doc_ids)

    # -- training primitives (all tensors on self.device)
    def _hs_tables(self):
        L = max(len(v.codes) for v in self.vocab.by_index)
        n = self.vocab.numWords()
        codes = torch.zeros(n, L)
        points = torch.zeros(n, L, dtype=torch.long)
        mask = torch.zeros(n, L)
        for i, v in enumerate(self.vocab.by_index):
            k = len(v.codes)
            codes[i, :k] = torch.tensor(v.codes, dtype=torch.float32)
            points[i, :k] = torch.tensor(v.points, dtype=torch.long)
            mask[i, :k] = 1.0
        return codes.to(self.device), points.to(self.device), mask.to(self.device)

    def _neg_table(self):
        f = torch.tensor([0.0 if v.is_label else v.count for v in self.vocab.by_index], dtype=torch.float64) ** 0.75
        return (f / f.sum()).float().to(self.device)

    def _output_step(self, h, target, lr, gen):
        """Updates the output layers for hidden vectors ``h`` [B,D] predicting ``target`` [B]; returns dL/dh scaled by -lr
        (i.e. the amount to add to the input vectors)."""
        lt = self.lookupTable
        dh = torch.zeros_like(h)
        if self.useHierarchicSoftmax:
            codes, points, mask = self._hs
            p, c, m = points[target], codes[target], mask[target]                      # [B,L]
            w = lt.syn1[p]                                                              # [B,L,D]
            f = torch.sigmoid(torch.einsum("bd,bld->bl", h, w))
            g = (1.0 - c - f) * m * lr
            dh += torch.einsum("bl,bld->bd", g, w)
            _scatter_add(lt.syn1, p.reshape(-1), (g.unsqueeze(-1) * h.unsqueeze(1)).reshape(-1, h.shape[1]))
        if self.negativeSample > 0:
            K = int(self.negativeSample)
            neg = torch.multinomial(self._neg, target.numel() * K, replacement=True, generator=gen).reshape(-1, K)
            tg = torch.cat([target.unsqueeze(1), neg], 1)                               # [B,1+K]
            lab = torch.zeros_like(tg, dtype=h.dtype)
            lab[:, 0] = 1.0
            valid = torch.ones_like(lab)
            valid[:, 1:] = (neg != target.unsqueeze(1)).to(h.dtype)
            w = lt.syn1Neg[tg]
            f = torch.sigmoid(torch.einsum("bd,bkd->bk", h, w))
            g = (lab - f) * valid * lr
            dh += torch.einsum("bk,bkd->bd", g, w)
            _scatter_add(lt.syn1Neg, tg.reshape(-1), (g.unsqueeze(-1) * h.unsqueeze(1)).reshape(-1, h.shape[1]))
        return dh

    def _native_tables(self):
        """Index tables in the form the batch kernel takes (``csrc/nlp_kernels.cu``), or None when the tables are not fp32 CUDA
        tensors: Huffman points with -1 padding, int8 codes, and a unigram^0.75 sample table of 2^20 entries."""
        lt = self.lookupTable
        if not (lt.syn0.is_cuda and lt.syn0.dtype == torch.float32) or getattr(self, "useTorchKernels", False):
            return None
        from ..ops import native
        if not native.available():
            return None
        t = getattr(self, "_native_tab", None)
        if t is None:
            t = {}
            if self.useHierarchicSoftmax:
                codes, points, mask = self._hs
                t["points"] = torch.where(mask > 0, points, torch.full_like(points, -1)).to(torch.int32)
                t["codes"] = codes.to(torch.int8)
            if self.negativeSample > 0:
                cdf = torch.cumsum(self._neg.double(), 0)
                u = (torch.arange(1 << 20, device=cdf.device, dtype=torch.float64) + 0.5) / float(1 << 20)
                t["neg"] = torch.searchsorted(cdf, u).clamp(max=cdf.numel() - 1).to(torch.int32)
            self._native_tab = t
        return t

    def _native_step(self, tab, rows_in, center, context, lr, gen):
        """One kernel launch for a batch: skip-gram (``rows_in`` = input rows of syn0, ``context`` None) or CBOW (``context`` [B, W])."""
        from ..ops import native
        lt = self.lookupTable
        hs, ns = self.useHierarchicSoftmax, self.negativeSample > 0
        rnd = torch.randint(0, 1 << 62, (center.numel(),), device=center.device, generator=gen)
        return native.w2v_batch(lt.syn0, lt.syn1 if hs else None, lt.syn1Neg if ns else None, tab.get("neg"), rows_in,
                                center if ns else None, tab["points"][center] if hs else None, tab["codes"][center] if hs else None,
                                context, torch.tensor([lr], dtype=torch.float32, device=center.device), rnd,
                                int(self.negativeSample) if ns else 0, True)

    def _pairs(self, ids, sent, gen):
        """(center position, context position) pairs with per-center dynamic windows and subsampling."""
        n = ids.numel()
        keep = torch.ones(n, dtype=torch.bool, device=ids.device)
        if self.sampling and self.sampling > 0:
            freq = torch.tensor([v.count for v in self.vocab.by_index], device=ids.device) / max(self.vocab.total, 1.0)
            f = freq[ids]
            prob = (torch.sqrt(f / self.sampling) + 1) * (self.sampling / f)
            keep = torch.rand(n, device=ids.device, generator=gen) < prob
        pos = keep.nonzero().squeeze(1)
        ids_k, sent_k = ids[pos], sent[pos]
        m = ids_k.numel()
        b = torch.randint(1, self.windowSize + 1, (m,), device=ids.device, generator=gen)
        cs, xs = [], []
        ar = torch.arange(m, device=ids.device)
        for d in range(-self.windowSize, self.windowSize + 1):
            if d == 0:
                continue
            j = ar + d
            ok = (j >= 0) & (j < m) & (abs(d) <= b)
            jj = j.clamp(0, max(m - 1, 0))
            ok &= sent_k[jj] == sent_k
            cs.append(ar[ok])
            xs.append(jj[ok])
        return ids_k, sent_k, torch.cat(cs), torch.cat(xs)

    def _train_elements(self, ids, sent, gen, lr_fn, progress):
        lt = self.lookupTable
        tab = self._native_tables()
        for _ in range(max(self.iterations, 1)):
            ids_k, sent_k, c, x = self._pairs(ids, sent, gen)
            if c.numel() == 0:
                continue
            if self.elementsLearningAlgorithm.lower() == "cbow":
                # group contexts per centre: padded [M, 2w] matrix
                m, W = ids_k.numel(), 2 * self.windowSize
                order = torch.argsort(c, stable=True)
                c_s, x_s = c[order], x[order]
                first = torch.searchsorted(c_s, torch.arange(m, device=c.device))
                slot = torch.arange(c_s.numel(), device=c.device) - first[c_s]
                ctx = torch.full((m, W), -1, dtype=torch.long, device=c.device)
                ctx[c_s, slot.clamp(max=W - 1)] = ids_k[x_s]
                has = (ctx >= 0).any(1).nonzero().squeeze(1)
                perm = has[torch.randperm(has.numel(), device=c.device, generator=gen)]
                for s in range(0, perm.numel(), self.batchSize):
                    rows = perm[s:s + self.batchSize]
                    cm = ctx[rows]
                    if tab is not None and self._native_step(tab, ids_k[rows], ids_k[rows], cm, lr_fn(progress[0]), gen):
                        progress[0] += rows.numel()
                        continue
                    msk = (cm >= 0).to(lt.syn0.dtype)
                    vecs = lt.syn0[cm.clamp(min=0)] * msk.unsqueeze(-1)
                    cnt = msk.sum(1, keepdim=True).clamp(min=1)
                    h = vecs.sum(1) / cnt
                    lr = lr_fn(progress[0])
                    dh = self._output_step(h, ids_k[rows], lr, gen)
                    upd = (dh / cnt).unsqueeze(1) * msk.unsqueeze(-1)
                    _scatter_add(lt.syn0, cm.clamp(min=0).reshape(-1), upd.reshape(-1, h.shape[1]))
                    progress[0] += rows.numel()
            else:
                perm = torch.randperm(c.numel(), device=c.device, generator=gen)
                for s in range(0, perm.numel(), self.batchSize):
                    sel = perm[s:s + self.batchSize]
                    center, context = ids_k[c[sel]], ids_k[x[sel]]
                    # skip-gram as in word2vec.c: the context word's vector is the input, the centre word the target
                    if tab is not None and self._native_step(tab, context, center, None, lr_fn(progress[0]), gen):
                        progress[0] += sel.numel() / (2.0 * self.windowSize)
                        continue
                    h = lt.syn0[context]
                    lr = lr_fn(progress[0])
                    dh = self._output_step(h, center, lr, gen)
                    _scatter_add(lt.syn0, context, dh)
                    progress[0] += sel.numel() / (2.0 * self.windowSize)

    def fit(self):
        if self.vocab is None or self.lookupTable is None:
            self.buildVocab()
        ids, sent, doc_ids = self._corpus_tensors()
        gen = torch.Generator(device=self.device).manual_seed(int(self.seed))
        if self.useHierarchicSoftmax:
            self._hs = self._hs_tables()
            self._native_tab = None
        if self.negativeSample > 0:
            self._neg = self._neg_table()
        total = max(ids.numel() * self.epochs * max(self.iterations, 1), 1)
        lr_fn = lambda done: max(self.minLearningRate, self.learningRate * (1.0 - done / total))
        progress = [0.0]
        for _ in range(self.epochs):
            if self.trainElementsRepresentation and ids.numel():
                self._train_elements(ids, sent, gen, lr_fn, progress)
            if self.trainSequencesRepresentation and any(doc_ids):
                self._train_sequences(ids, sent, doc_ids, gen, lr_fn)
        return self

    def _train_sequences(self, ids, sent, doc_ids, gen, lr_fn):
        pass

    # -- queries (WordVectors interface)
    def vocab_(self): return self.vocab
    def getVocab(self): return self.vocab
    def getLookupTable(self): return self.lookupTable
    lookupTable_ = getLookupTable
    def hasWord(self, w): return self.vocab is not None and self.vocab.containsWord(w)
    def indexOf(self, w): return self.vocab.indexOf(w)
    def getLayerSize(self): return self.layerSize

    def getWordVectorMatrix(self, w):
        i = self.vocab.indexOf(w)
        if i < 0:
            if self.useUnknown:
                i = self.vocab.indexOf(self.unknownElement)
            else:
                return None
        return INDArray(self.lookupTable.syn0[i])

    def getWordVector(self, w):
        v = self.getWordVectorMatrix(w)
        return None if v is None else v.t.tolist()

    def getWordVectors(self, words):
        idx = [self.vocab.indexOf(w) for w in words if self.vocab.indexOf(w) >= 0]
        return INDArray(self.lookupTable.syn0[torch.tensor(idx, dtype=torch.long, device=self.device)])

    def getWordVectorsMean(self, words): return INDArray(self.getWordVectors(words).t.mean(0))

    def _normed(self, restrict_words=True):
        s = self.lookupTable.syn0
        return s / s.norm(dim=1, keepdim=True).clamp(min=1e-12)

    def similarity(self, a, b):
        va, vb = self.getWordVectorMatrix(a), self.getWordVectorMatrix(b)
        if va is None or vb is None:
            return float("nan")
        return float(torch.nn.functional.cosine_similarity(va.t, vb.t, dim=0))

    def _nearest_to_vector(self, v, n, exclude=()):
        sims = self._normed() @ (v / v.norm().clamp(min=1e-12))
        is_label = torch.tensor([x.is_label for x in self.vocab.by_index], device=sims.device)
        sims = sims.masked_fill(is_label, -2.0)
        for w in exclude:
            i = self.vocab.indexOf(w)
            if i >= 0:
                sims[i] = -2.0
        k = min(n, int((sims > -2.0).sum()))
        top = sims.topk(k).indices.tolist() if k > 0 else []
        return [self.vocab.wordAtIndex(i) for i in top]

    def wordsNearest(self, positive, negative=None, n=10):
        if isinstance(negative, int):
            negative, n = None, negative
        if isinstance(positive, INDArray) or isinstance(positive, torch.Tensor):
            return self._nearest_to_vector(positive.t if isinstance(positive, INDArray) else positive, n)
        pos = [positive] if isinstance(positive, str) else list(positive)
        neg = list(negative or [])
        nm = self._normed()
        v = sum(nm[self.vocab.indexOf(w)] for w in pos if self.hasWord(w))
        for w in neg:
            if self.hasWord(w):
                v = v - nm[self.vocab.indexOf(w)]
        return self._nearest_to_vector(v, n, exclude=pos + neg)

    def wordsNearestSum(self, positive, negative=None, n=10): return self.wordsNearest(positive, negative, n)
    def similarWordsInVocabTo(self, word, accuracy):
        import difflib
        return [w for w in self.vocab.words_() if difflib.SequenceMatcher(None, w, word).ratio() >= accuracy]


def _builder_for(cls):
    class Builder:
        def __init__(self): self.kw = {}
        def __getattr__(self, k):
            if k.startswith("_") or k == "kw":
                raise AttributeError(k)
            def s(*v):
                self.kw[k] = v[0] if len(v) == 1 else list(v)
                return self
            return s
        def build(self): return cls(**self.kw)
    return Builder


class Word2Vec(SequenceVectors):
    def __init__(self, **kw):
        kw.setdefault("trainSequencesRepresentation", False)
        super().__init__(**kw)


Word2Vec.Builder = _builder_for(Word2Vec)


class ParagraphVectors(SequenceVectors):
    """Document embeddings: labels are extra rows of ``syn0``.  DBOW: the document vector alone predicts each word of
    the document; DM: the mean of document vector and context words predicts the centre word."""

    def __init__(self, **kw):
        kw.setdefault("trainElementsRepresentation", kw.pop("trainWordVectors", True))
        it = kw.get("iterate")
        if isinstance(it, (list, tuple)) and it and isinstance(it[0], str):
            src = kw.get("labelsSource") or LabelsSource("DOC_")
            kw["iterate"] = [LabelledDocument(s, [src.nextLabel()]) for s in it]
            kw["labelsSource"] = src
        elif isinstance(it, SentenceIterator):
            kw["iterate"] = list(SentenceIteratorConverter(it, kw.get("labelsSource")))
        super().__init__(**kw)

    def _doc_pairs(self, ids, sent, doc_ids):
        docs, words = [], []
        counts = torch.bincount(sent, minlength=len(doc_ids)).tolist() if sent.numel() else [0] * len(doc_ids)
        start = 0
        for s, labs in enumerate(doc_ids):
            n = counts[s] if s < len(counts) else 0
            for l in labs:
                if l >= 0 and n:
                    docs.append(torch.full((n,), l, dtype=torch.long, device=ids.device))
                    words.append(ids[start:start + n])
            start += n
        if not docs:
            return None, None
        return torch.cat(docs), torch.cat(words)

    def _train_sequences(self, ids, sent, doc_ids, gen, lr_fn):
        lt = self.lookupTable
        d, w = self._doc_pairs(ids, sent, doc_ids)
        if d is None:
            return
        for _ in range(max(self.iterations, 1)):
            perm = torch.randperm(d.numel(), device=d.device, generator=gen)
            for s in range(0, perm.numel(), self.batchSize):
                sel = perm[s:s + self.batchSize]
                h = lt.syn0[d[sel]]
                dh = self._output_step(h, w[sel], lr_fn(0), gen)
                _scatter_add(lt.syn0, d[sel], dh)

    def inferVector(self, text, learningRate=0.025, minLearningRate=1e-4, iterations=20):
        toks = text if isinstance(text, (list, tuple)) else self.tokenizerFactory.create(text.getContent() if hasattr(text, "getContent") else text).getTokens()
        idx = [self.vocab.indexOf(t) for t in toks]
        idx = torch.tensor([i for i in idx if i >= 0], dtype=torch.long, device=self.device)
        g = torch.Generator(device=self.device).manual_seed(int(self.seed) + 1)
        v = ((torch.rand(1, self.layerSize, device=self.device, generator=g) - 0.5) / self.layerSize)
        if idx.numel() == 0:
            return INDArray(v[0])
        lt = self.lookupTable
        saved = (None if lt.syn1 is None else lt.syn1.clone(), None if lt.syn1Neg is None else lt.syn1Neg.clone())
        if self.useHierarchicSoftmax and not hasattr(self, "_hs"):
            self._hs = self._hs_tables()
            self._native_tab = None
        if self.negativeSample > 0 and not hasattr(self, "_neg"):
            self._neg = self._neg_table()
        for it in range(iterations):
            lr = max(minLearningRate, learningRate * (1 - it / iterations))
            h = v.expand(idx.numel(), -1)
            dh = self._output_step(h, idx, lr, g)
            v = v + dh.sum(0, keepdim=True)
        if saved[0] is not None:
            lt.syn1.copy_(saved[0])
        if saved[1] is not None:
            lt.syn1Neg.copy_(saved[1])
        return INDArray(v[0])

    def _label_rows(self):
        idx = [v.index for v in self.vocab.by_index if v.is_label]
        return idx, self.lookupTable.syn0[torch.tensor(idx, dtype=torch.long, device=self.device)]

    def nearestLabels(self, text_or_vec, n=5):
        v = text_or_vec.t if isinstance(text_or_vec, INDArray) else (text_or_vec if isinstance(text_or_vec, torch.Tensor) else self.inferVector(text_or_vec).t)
        idx, rows = self._label_rows()
        sims = torch.nn.functional.cosine_similarity(rows, v.unsqueeze(0), dim=1)
        top = sims.topk(min(n, len(idx))).indices.tolist()
        return [self.vocab.wordAtIndex(idx[i]) for i in top]

    def predict(self, text): return self.nearestLabels(text, 1)[0]
    def predictSeveral(self, text, n): return self.nearestLabels(text, n)

    def similarityToLabel(self, text, label):
        v = self.inferVector(text).t
        return float(torch.nn.functional.cosine_similarity(v, self.lookupTable.syn0[self.vocab.indexOf(label)], dim=0))

    def getLabelsSource(self): return self.labelsSource


ParagraphVectors.Builder = _builder_for(ParagraphVectors)


# ----------------------------------------------------------------------------- serialisation
class WordVectorSerializer:
    """Text (``word v1 v2 ...``), Google binary and the zip model format (``syn0.txt``, ``syn1.txt``, ``syn1Neg.txt``,
    ``codes.txt``, ``huffman.txt``, ``frequencies.txt``, ``config.json``) of ``WordVectorSerializer.java``."""

    @staticmethod
    def writeWordVectors(model, path):
        syn0 = model.lookupTable.syn0.detach().cpu()
        with open(path, "w", encoding="utf-8") as f:
            f.write(f"{syn0.shape[0]} {syn0.shape[1]}\n")
            for v in model.vocab.by_index:
                f.write(v.word.replace(" ", "_") + " " + " ".join(f"{x:.6f}" for x in syn0[v.index].tolist()) + "\n")

    @staticmethod
    def loadTxtVectors(path, device="cpu"):
        words, rows = [], []
        with open(path, encoding="utf-8") as f:
            first = f.readline().split()
            if len(first) != 2 or not all(t.isdigit() for t in first):
                words.append(first[0])
                rows.append([float(x) for x in first[1:]])
            for line in f:
                p = line.rstrip("\n").split(" ")
                if len(p) < 2:
                    continue
                words.append(p[0])
                rows.append([float(x) for x in p[1:]])
        return WordVectorSerializer._from_rows(words, torch.tensor(rows, dtype=torch.float32), device)

    readWord2VecModel_txt = loadTxtVectors

    @staticmethod
    def _from_rows(words, mat, device="cpu", counts=None):
        m = Word2Vec(layerSize=mat.shape[1], device=device, iterate=[])
        vc = VocabCache()
        for i, w in enumerate(words):
            vw = VocabWord(w, counts[i] if counts else float(len(words) - i), i)
            vc.words[w] = vw
            vc.by_index.append(vw)
        m.vocab = vc
        m.lookupTable = InMemoryLookupTable(vc, mat.shape[1], 0, device)
        m.lookupTable.syn0 = mat.to(device)
        return m

    @staticmethod
    def writeBinary(model, path):
        syn0 = model.lookupTable.syn0.detach().cpu().float()
        with open(path, "wb") as f:
            f.write(f"{syn0.shape[0]} {syn0.shape[1]}\n".encode())
            for v in model.vocab.by_index:
                f.write(v.word.encode("utf-8") + b" " + syn0[v.index].numpy().astype("<f4").tobytes() + b"\n")

    @staticmethod
    def readBinaryModel(path, device="cpu"):
        with open(path, "rb") as f:
            n, d = (int(x) for x in f.readline().split())
            words, mat = [], np.zeros((n, d), dtype=np.float32)
            for i in range(n):
                w = bytearray()
                while True:
                    c = f.read(1)
                    if c in (b" ", b""):
                        break
                    if c != b"\n":
                        w += c
                words.append(w.decode("utf-8", errors="replace"))
                mat[i] = np.frombuffer(f.read(4 * d), dtype="<f4")
        return WordVectorSerializer._from_rows(words, torch.from_numpy(mat), device)

    @staticmethod
    def writeWord2VecModel(model, path):
        lt, vc = model.lookupTable, model.vocab
        def mat_lines(m): return "\n".join(" ".join(f"{x:.8g}" for x in row) for row in m.detach().cpu().tolist())
        with zipfile.ZipFile(path, "w", zipfile.ZIP_DEFLATED) as z:
            z.writestr("syn0.txt", f"{vc.numWords()} {model.layerSize} {vc.numWords()}\n" +
                       "\n".join("B64:" + __import__("base64").b64encode(v.word.encode()).decode() + " " +
                                 " ".join(f"{x:.8g}" for x in lt.syn0[v.index].tolist()) for v in vc.by_index))
            if lt.syn1 is not None:
                z.writestr("syn1.txt", mat_lines(lt.syn1))
            if lt.syn1Neg is not None:
                z.writestr("syn1Neg.txt", mat_lines(lt.syn1Neg))
            z.writestr("codes.txt", "\n".join(v.word + " " + " ".join(str(c) for c in v.codes) for v in vc.by_index))
            z.writestr("huffman.txt", "\n".join(v.word + " " + " ".join(str(p) for p in v.points) for v in vc.by_index))
            z.writestr("frequencies.txt", "\n".join(f"{v.word} {v.count} {1 if v.is_label else 0}" for v in vc.by_index))
            cfg = {k: getattr(model, k) for k in ("minWordFrequency", "iterations", "epochs", "layerSize", "seed", "windowSize", "learningRate",
                                                  "minLearningRate", "negativeSample", "useHierarchicSoftmax", "sampling", "batchSize",
                                                  "elementsLearningAlgorithm", "sequenceLearningAlgorithm", "useUnknown", "unknownElement")}
            cfg["modelType"] = type(model).__name__
            z.writestr("config.json", json.dumps(cfg))

    writeParagraphVectors = writeWord2VecModel

    @staticmethod
    def readWord2VecModel(path, device="cpu"):
        import base64
        if not zipfile.is_zipfile(path):
            try:
                return WordVectorSerializer.loadTxtVectors(path, device)
            except (UnicodeDecodeError, ValueError):
                return WordVectorSerializer.readBinaryModel(path, device)
        with zipfile.ZipFile(path) as z:
            cfg = json.loads(z.read("config.json"))
            mt = cfg.pop("modelType", "Word2Vec")
            model = (ParagraphVectors if mt == "ParagraphVectors" else Word2Vec)(iterate=[], device=device, **cfg)
            lines = z.read("syn0.txt").decode().split("\n")
            words, rows = [], []
            for l in lines[1:]:
                p = l.split(" ")
                w = p[0]
                words.append(base64.b64decode(w[4:]).decode() if w.startswith("B64:") else w)
                rows.append([float(x) for x in p[1:]])
            freq = {}
            for l in z.read("frequencies.txt").decode().split("\n"):
                p = l.rsplit(" ", 2)
                freq[p[0]] = (float(p[1]), p[2] == "1")
            vc = VocabCache()
            for i, w in enumerate(words):
                vw = VocabWord(w, freq.get(w, (1.0, False))[0], i, freq.get(w, (1.0, False))[1])
                vc.words[w] = vw
                vc.by_index.append(vw)
                vc.total += 0 if vw.is_label else vw.count
            for name, attr in (("codes.txt", "codes"), ("huffman.txt", "points")):
                for l in z.read(name).decode().split("\n"):
                    p = l.split(" ")
                    if p[0] in vc.words:
                        setattr(vc.words[p[0]], attr, [int(x) for x in p[1:] if x != ""])
            model.vocab = vc
            lt = InMemoryLookupTable(vc, cfg["layerSize"], cfg["seed"], device)
            lt.syn0 = torch.tensor(rows, dtype=torch.float32, device=device)
            names = z.namelist()
            rd = lambda n: torch.tensor([[float(x) for x in l.split(" ")] for l in z.read(n).decode().split("\n") if l], dtype=torch.float32, device=device)
            lt.syn1 = rd("syn1.txt") if "syn1.txt" in names else None
            lt.syn1Neg = rd("syn1Neg.txt") if "syn1Neg.txt" in names else None
            model.lookupTable = lt
            return model

    readParagraphVectors = readWord2VecModel
