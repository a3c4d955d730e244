"""``BertIterator`` and ``BertMaskedLMMasker`` (``deeplearning4j-nlp/.../iterator/BertIterator.java``,
``iterator/bert/BertMaskedLMMasker.java``): turns sentences (optionally sentence pairs / labelled sentences) into
MultiDataSets of token indices, attention masks and optional segment ids for BERT pre-training (masked LM) or
sequence classification."""
from __future__ import annotations

import random

import torch

from ..data.dataset import MultiDataSet


class BertMaskedLMMasker:
    DEFAULT_MASK_PROB = 0.15
    DEFAULT_MASK_TOKEN_PROB = 0.8
    DEFAULT_RANDOM_WORD_PROB = 0.1

    def __init__(self, rng=None, maskProb=DEFAULT_MASK_PROB, maskTokenProb=DEFAULT_MASK_TOKEN_PROB, randomTokenProb=DEFAULT_RANDOM_WORD_PROB):
        if not 0 < maskProb < 1:
            raise ValueError(f"Probability must be between 0 and 1, got {maskProb}")
        if maskTokenProb + randomTokenProb > 1.0:
            raise ValueError("Sum of maskTokenProb and randomTokenProb must be <= 1.0")
        self.r = rng if rng is not None else random.Random(12345)
        self.maskProb, self.maskTokenProb, self.randomTokenProb = maskProb, maskTokenProb, randomTokenProb

    def maskSequence(self, tokens, maskToken, vocabWords):
        """Returns (masked tokens, isMasked flags): each token is selected with ``maskProb``; a selected token becomes the
        mask token (80 %), a random vocabulary word (10 %) or stays unchanged (10 %)."""
        out, flags = [], []
        for t in tokens:
            if self.r.random() < self.maskProb:
                u = self.r.random()
                if u < self.maskTokenProb:
                    out.append(maskToken)
                elif u < self.maskTokenProb + self.randomTokenProb:
                    out.append(vocabWords[self.r.randrange(len(vocabWords))])
                else:
                    out.append(t)
                flags.append(True)
            else:
                out.append(t)
                flags.append(False)
        return out, flags


class BertIterator:
    class Task:
        UNSUPERVISED = "UNSUPERVISED"
        SEQ_CLASSIFICATION = "SEQ_CLASSIFICATION"

    class LengthHandling:
        FIXED_LENGTH = "FIXED_LENGTH"
        ANY_LENGTH = "ANY_LENGTH"
        CLIP_ONLY = "CLIP_ONLY"

    class FeatureArrays:
        INDICES_MASK = "INDICES_MASK"
        INDICES_MASK_SEGMENTID = "INDICES_MASK_SEGMENTID"

    class UnsupervisedLabelFormat:
        RANK2_IDX = "RANK2_IDX"
        RANK3_NCL = "RANK3_NCL"
        RANK3_LNC = "RANK3_LNC"

    def __init__(self, task, tokenizerFactory, sentenceProvider=None, sentencePairProvider=None, lengthHandling="FIXED_LENGTH", maxTokens=128,
                 minibatchSize=32, padMinibatches=False, featureArrays="INDICES_MASK", vocabMap=None, masker=None,
                 unsupervisedLabelFormat="RANK2_IDX", maskToken="[MASK]", prependToken="[CLS]", appendToken=None, preProcessor=None):
        self.task, self.tf = task, tokenizerFactory
        self.provider, self.pairProvider = sentenceProvider, sentencePairProvider
        self.lengthHandling, self.maxTokens, self.minibatchSize, self.padMinibatches = lengthHandling, int(maxTokens), int(minibatchSize), padMinibatches
        self.featureArrays = featureArrays
        self.vocabMap = vocabMap or tokenizerFactory.getVocab()
        self.vocabWords = [w for w, _ in sorted(self.vocabMap.items(), key=lambda kv: kv[1])]
        self.masker = masker or BertMaskedLMMasker()
        self.labelFormat, self.maskToken, self.prependToken, self.appendToken = unsupervisedLabelFormat, maskToken, prependToken, appendToken
        self.preProcessor = preProcessor
        self._labels = None
        self.reset()

    class Builder:
        def __init__(self): self.kw = {}
        def task(self, t): self.kw["task"] = t; return self
        def tokenizer(self, t): self.kw["tokenizerFactory"] = t; return self
        def lengthHandling(self, lh, maxLength): self.kw["lengthHandling"], self.kw["maxTokens"] = lh, maxLength; return self
        def minibatchSize(self, n): self.kw["minibatchSize"] = n; return self
        def padMinibatches(self, b): self.kw["padMinibatches"] = b; return self
        def featureArrays(self, f): self.kw["featureArrays"] = f; return self
        def vocabMap(self, m): self.kw["vocabMap"] = m; return self
        def masker(self, m): self.kw["masker"] = m; return self
        def unsupervisedLabelFormat(self, f): self.kw["unsupervisedLabelFormat"] = f; return self
        def maskToken(self, t): self.kw["maskToken"] = t; return self
        def prependToken(self, t): self.kw["prependToken"] = t; return self
        def appendToken(self, t): self.kw["appendToken"] = t; return self
        def sentenceProvider(self, p): self.kw["sentenceProvider"] = p; return self
        def sentencePairProvider(self, p): self.kw["sentencePairProvider"] = p; return self
        def preProcessor(self, p): self.kw["preProcessor"] = p; return self
        def build(self): return BertIterator(**self.kw)

    @staticmethod
    def builder(): return BertIterator.Builder()

    # -- iteration
    def reset(self):
        src = self.pairProvider if self.pairProvider is not None else self.provider
        if hasattr(src, "reset"):
            src.reset()
        self._it = iter(self._items(src))
        self._peek = next(self._it, None)

    def _items(self, src):
        if src is None:
            return
        for item in src:
            if hasattr(item, "getContent"):
                yield (item.getContent(), None, item.getLabel())
            elif isinstance(item, (tuple, list)) and self.pairProvider is not None:
                yield (item[0], item[1], item[2] if len(item) > 2 else None)
            elif isinstance(item, (tuple, list)):
                yield (item[0], None, item[1] if len(item) > 1 else None)
            else:
                yield (item, None, None)

    def hasNext(self): return self._peek is not None
    def resetSupported(self): return True
    def asyncSupported(self): return True
    def batch(self): return self.minibatchSize

    def __iter__(self):
        self.reset()
        while self.hasNext():
            yield self.next()

    def _tokenize(self, a, b):
        ta = self.tf.create(a).getTokens()
        seg = None
        if self.prependToken:
            ta = [self.prependToken] + ta
        if b is not None:
            sep = self.appendToken or "[SEP]"
            tb = self.tf.create(b).getTokens()
            budget = self.maxTokens - 2 if self.lengthHandling != self.LengthHandling.ANY_LENGTH else 1 << 30
            while len(ta) + len(tb) > budget and (len(ta) > 1 or len(tb) > 0):      # trim the longer side first
                if len(ta) > len(tb):
                    ta.pop()
                else:
                    tb.pop()
            toks = ta + [sep] + tb + [sep]
            seg = [0] * (len(ta) + 1) + [1] * (len(tb) + 1)
        else:
            toks = ta + ([self.appendToken] if self.appendToken else [])
        if self.lengthHandling != self.LengthHandling.ANY_LENGTH and len(toks) > self.maxTokens:
            toks = toks[:self.maxTokens]
            if self.appendToken and b is None:
                toks[-1] = self.appendToken
            if seg is not None:
                seg = seg[:self.maxTokens]
        return toks, seg

    def next(self, n=None):
        n = n or self.minibatchSize
        rows = []
        while self._peek is not None and len(rows) < n:
            rows.append(self._peek)
            self._peek = next(self._it, None)
        return self._make(rows)

    __next__ = next

    def featurizeSentences(self, sentences):
        return self._make([(s, None, None) for s in sentences], features_only=True)

    def featurizeSentencePairs(self, pairs):
        return self._make([(a, b, None) for a, b in pairs], features_only=True)

    def _make(self, rows, features_only=False):
        unk = self.vocabMap.get("[UNK]", 0)
        toks, segs, masked_flags, originals = [], [], [], []
        for a, b, _ in rows:
            t, s = self._tokenize(a, b)
            originals.append(t)
            if self.task == self.Task.UNSUPERVISED and not features_only:
                t2, fl = self.masker.maskSequence(t, self.maskToken, self.vocabWords)
                if self.prependToken and t and t[0] == self.prependToken:          # never mask the classifier token
                    t2[0], fl[0] = t[0], False
                toks.append(t2)
                masked_flags.append(fl)
            else:
                toks.append(t)
            segs.append(s)
        longest = max((len(t) for t in toks), default=0)
        T = self.maxTokens if self.lengthHandling == self.LengthHandling.FIXED_LENGTH else min(longest, self.maxTokens) \
            if self.lengthHandling == self.LengthHandling.CLIP_ONLY else longest
        N = len(rows)
        Np = self.minibatchSize if (self.padMinibatches and N < self.minibatchSize) else N
        idx = torch.zeros(Np, T, dtype=torch.int64)
        mask = torch.zeros(Np, T, dtype=torch.float32)
        segid = torch.zeros(Np, T, dtype=torch.int64)
        for i, t in enumerate(toks):
            ids = [self.vocabMap.get(x, unk) for x in t[:T]]
            idx[i, :len(ids)] = torch.tensor(ids, dtype=torch.int64)
            mask[i, :len(ids)] = 1.0
            if segs[i] is not None:
                segid[i, :len(ids)] = torch.tensor(segs[i][:T], dtype=torch.int64)
        feats = [idx, segid] if self.featureArrays == self.FeatureArrays.INDICES_MASK_SEGMENTID else [idx]
        fmasks = [mask, None] if len(feats) == 2 else [mask]
        if features_only:
            return feats, fmasks
        if self.task == self.Task.UNSUPERVISED:
            lmask = torch.zeros(Np, T, dtype=torch.float32)
            lab_idx = torch.zeros(Np, T, dtype=torch.int64)
            for i, (orig, fl) in enumerate(zip(originals, masked_flags)):
                for j, (tok, m) in enumerate(zip(orig[:T], fl[:T])):
                    lab_idx[i, j] = self.vocabMap.get(tok, unk)
                    if m:
                        lmask[i, j] = 1.0
            if self.labelFormat == self.UnsupervisedLabelFormat.RANK2_IDX:
                labels = lab_idx
            else:
                V = len(self.vocabMap)
                oh = torch.nn.functional.one_hot(lab_idx, V).float()                  # [N, T, V]
                labels = oh.permute(0, 2, 1).contiguous() if self.labelFormat == self.UnsupervisedLabelFormat.RANK3_NCL else oh.permute(1, 0, 2).contiguous()
            mds = MultiDataSet(feats, [labels], fmasks, [lmask])
        else:
            if self._labels is None:
                src = self.provider if self.provider is not None else self.pairProvider
                self._labels = list(src.allLabels()) if hasattr(src, "allLabels") else sorted({str(r[2]) for r in rows if r[2] is not None})
            lab = torch.zeros(Np, len(self._labels))
            for i, (_, _, l) in enumerate(rows):
                if l is not None and str(l) in self._labels:
                    lab[i, self._labels.index(str(l))] = 1.0
            mds = MultiDataSet(feats, [lab], fmasks, None)
        if self.preProcessor is not None:
            self.preProcessor.preProcess(mds)
        return mds


class CollectionLabeledSentenceProvider:
    """(sentence, label) pairs from two parallel collections (``CollectionLabeledSentenceProvider.java``)."""

    def __init__(self, sentences, labels, rng=None):
        self.items = list(zip(sentences, labels))
        self.rng = rng
        self.labels = sorted({str(l) for l in labels})

    def __iter__(self):
        order = list(range(len(self.items)))
        if self.rng is not None:
            self.rng.shuffle(order)
        for i in order:
            yield self.items[i]

    def reset(self): pass
    def totalNumSentences(self): return len(self.items)
    def allLabels(self): return self.labels
    def numLabelClasses(self): return len(self.labels)


class CollectionLabeledPairSentenceProvider(CollectionLabeledSentenceProvider):
    def __init__(self, left, right, labels, rng=None):
        self.items = list(zip(left, right, labels))
        self.rng = rng
        self.labels = sorted({str(l) for l in labels})
