"""FastText: sub-word (character n-gram) embeddings and the bag-of-n-grams text classifier.

Parity: ``deeplearning4j-nlp/.../models/fasttext/FastText.java`` (builder options ``supervised / skipgram / cbow``, ``dim``,
``minCount``, ``wordNgrams``-less character n-grams ``minn / maxn``, ``bucket``, ``negativeSamples``, ``epochs``, ``lr``, label prefix
``__label__``; ``fit``, ``predict``, ``predictProbability``, ``getWordVector`` with out-of-vocabulary words composed from their
n-grams, ``wordsNearest``, ``similarity``, model save / load).  The reference delegates to the native fastText library; here the
model is trained with batched torch ops (on the GPU when one is given): a word is the mean of its own vector and the vectors of its
hashed n-grams (FNV-1a, as in fastText), skip-gram uses negative sampling from the unigram^0.75 table, the supervised mode averages
the token vectors of a line and trains a softmax layer over the labels.
"""
from __future__ import annotations

import io
import json
import zipfile

import numpy as np
import torch

from ..nd.ndarray import INDArray


def _fnv1a(s: str) -> int:
    h = 2166136261
    for b in s.encode("utf-8"):
        h = ((h ^ (b if b < 128 else b - 256)) & 0xFFFFFFFF) * 16777619 & 0xFFFFFFFF      # fastText casts bytes to int8 first
    return h


class FastText:
    LABEL_PREFIX = "__label__"

    def __init__(self, supervised=False, skipgram=True, cbow=False, dim=100, minCount=1, minn=3, maxn=6, bucket=200000, negativeSamples=5,
                 epochs=5, lr=0.05, windowSize=5, labelPrefix="__label__", seed=42, inputFile=None, iterator=None, device="cpu",
                 batchSize=2048, **_ignored):
        self.supervised, self.cbow = bool(supervised), bool(cbow) and not supervised
        self.dim, self.minCount, self.minn, self.maxn, self.bucket = int(dim), int(minCount), int(minn), int(maxn), int(bucket)
        self.negative, self.epochs, self.lr, self.window = int(negativeSamples), int(epochs), float(lr), int(windowSize)
        self.labelPrefix, self.seed, self.inputFile, self.iterator = labelPrefix, int(seed), inputFile, iterator
        self.device, self.batchSize = torch.device(device), int(batchSize)
        self.words, self.word_index, self.counts, self.labels = [], {}, [], []
        self.input = None          # [nwords + bucket, dim]
        self.output = None         # skip-gram: [nwords, dim]; supervised: [nlabels, dim]
        self._ngram_cache = {}

    # ------------------------------------------------------------------ builder
    class Builder:
        def __init__(self): self.kw = {}
        def __getattr__(self, k):
            def s(*v):
                self.kw[k] = v[0] if v else True
                return self
            return s
        def build(self): return FastText(**self.kw)

    @staticmethod
    def builder(): return FastText.Builder()

    # ------------------------------------------------------------------ corpus
    def _lines(self):
        if self.iterator is not None:
            it = self.iterator
            if hasattr(it, "reset"):
                it.reset()
            if hasattr(it, "hasNext"):
                while it.hasNext():
                    yield it.nextSentence() if hasattr(it, "nextSentence") else it.next()
            else:
                yield from it
        elif self.inputFile is not None:
            with open(self.inputFile, encoding="utf-8") as f:
                for line in f:
                    yield line.rstrip("\n")
        else:
            raise ValueError("FastText needs inputFile(...) or iterator(...)")

    def _subwords(self, word):
        """Row indices of a word: its own row (when in vocabulary) followed by its hashed character n-grams."""
        c = self._ngram_cache.get(word)
        if c is not None:
            return c
        rows = []
        wi = self.word_index.get(word)
        if wi is not None:
            rows.append(wi)
        if self.maxn > 0:
            w = "<" + word + ">"
            n_words = len(self.words)
            for n in range(self.minn, self.maxn + 1):
                for i in range(0, len(w) - n + 1):
                    g = w[i:i + n]
                    if n == 1 and (i == 0 or i == len(w) - 1):
                        continue
                    rows.append(n_words + _fnv1a(g) % self.bucket)
        self._ngram_cache[word] = rows
        return rows

    def _build_vocab(self, lines):
        cnt, lab = {}, {}
        for line in lines:
            for tok in line.split():
                if tok.startswith(self.labelPrefix):
                    lab[tok] = lab.get(tok, 0) + 1
                else:
                    cnt[tok] = cnt.get(tok, 0) + 1
        kept = sorted((w for w, c in cnt.items() if c >= self.minCount), key=lambda w: (-cnt[w], w))
        self.words, self.counts = kept, [cnt[w] for w in kept]
        self.word_index = {w: i for i, w in enumerate(kept)}
        self.labels = sorted(lab, key=lambda l: (-lab[l], l))
        self._ngram_cache.clear()

    def _bag(self, tokens):
        """(flat row indices, offsets) of a list of tokens for ``embedding_bag``-style means."""
        rows, offs = [], []
        for t in tokens:
            offs.append(len(rows))
            rows.extend(self._subwords(t))
        return rows, offs

    def _mean_rows(self, rows_list):
        """Mean input vector for each entry of ``rows_list`` (list of row-index lists)."""
        flat = [r for rows in rows_list for r in rows]
        lens = torch.tensor([max(len(r), 1) for r in rows_list], device=self.device, dtype=torch.float32)
        if not flat:
            return torch.zeros(len(rows_list), self.dim, device=self.device), None, lens
        idx = torch.tensor(flat, device=self.device)
        seg = torch.repeat_interleave(torch.arange(len(rows_list), device=self.device),
                                      torch.tensor([len(r) for r in rows_list], device=self.device))
        out = torch.zeros(len(rows_list), self.dim, device=self.device).index_add_(0, seg, self.input[idx])
        return out / lens[:, None], (idx, seg), lens

    # ------------------------------------------------------------------ training
    @staticmethod
    def _apply(table, idx, upd):
        """``table[idx] += upd`` where rows hit k times in the batch receive the sum damped by sqrt(k): plain sums of many
        duplicate updates (small vocabularies, large batches) overshoot, the per-row mean learns too slowly."""
        cnt = torch.bincount(idx, minlength=table.shape[0]).clamp_min(1).to(upd.dtype)
        table.index_add_(0, idx, upd / cnt[idx].sqrt()[:, None])

    def fit(self):
        lines = list(self._lines())
        self._build_vocab(lines)
        g = torch.Generator(device="cpu").manual_seed(self.seed)
        n_words = len(self.words)
        self.input = ((torch.rand(n_words + self.bucket, self.dim, generator=g) - 0.5) / self.dim).to(self.device)
        n_out = len(self.labels) if self.supervised else n_words
        self.output = torch.zeros(max(n_out, 1), self.dim, device=self.device)
        if self.supervised:
            self._fit_supervised(lines, g)
        else:
            self._fit_unsupervised(lines, g)
        return self

    def _fit_supervised(self, lines, g):
        data = []
        for line in lines:
            toks = line.split()
            labs = [self.labels.index(t) for t in toks if t.startswith(self.labelPrefix) and t in self.labels]
            words = [t for t in toks if not t.startswith(self.labelPrefix)]
            rows = [r for w in words for r in self._subwords(w)]
            if labs and rows:
                data.append((rows, labs[0]))
        if not data:
            raise ValueError("no labelled lines (labels start with %r)" % self.labelPrefix)
        total = self.epochs * len(data)
        seen = 0
        for _ in range(self.epochs):
            perm = torch.randperm(len(data), generator=g).tolist()
            for s in range(0, len(perm), self.batchSize):
                batch = [data[i] for i in perm[s:s + self.batchSize]]
                lr = self.lr * max(1.0 - seen / total, 1e-4)
                h, (idx, seg), lens = self._mean_rows([b[0] for b in batch])
                y = torch.tensor([b[1] for b in batch], device=self.device)
                logits = h @ self.output.t()
                p = torch.softmax(logits, -1)
                p[torch.arange(len(batch), device=self.device), y] -= 1.0          # d loss / d logits
                gh = p @ self.output                                              # [B, dim]
                self.output -= lr * (p.t() @ h) / 1.0
                self.input.index_add_(0, idx, -(lr * gh / lens[:, None])[seg])
                seen += len(batch)

    def _fit_unsupervised(self, lines, g):
        ids = [[self.word_index[t] for t in line.split() if t in self.word_index] for line in lines]
        ids = [s for s in ids if len(s) > 1]
        if not ids:
            return
        freq = torch.tensor(self.counts, dtype=torch.float64) ** 0.75
        neg_table = (freq / freq.sum()).float()
        pairs = []
        for sent in ids:
            for i, c in enumerate(sent):
                lo, hi = max(0, i - self.window), min(len(sent), i + self.window + 1)
                if self.cbow:
                    ctx = [sent[j] for j in range(lo, hi) if j != i]
                    if ctx:
                        pairs.append((ctx, c))
                else:
                    for j in range(lo, hi):
                        if j != i:
                            pairs.append(([c], sent[j]))
        total = self.epochs * len(pairs)
        seen = 0
        sub = [self._subwords(w) for w in self.words]
        for _ in range(self.epochs):
            perm = torch.randperm(len(pairs), generator=g).tolist()
            for s in range(0, len(perm), self.batchSize):
                batch = [pairs[i] for i in perm[s:s + self.batchSize]]
                lr = self.lr * max(1.0 - seen / total, 1e-4)
                h, (idx, seg), lens = self._mean_rows([[r for w in b[0] for r in sub[w]] for b in batch])
                B = len(batch)
                tgt = torch.tensor([b[1] for b in batch], device=self.device)
                neg = torch.multinomial(neg_table, B * self.negative, replacement=True, generator=g).to(self.device).view(B, self.negative)
                cand = torch.cat([tgt[:, None], neg], 1)                           # [B, 1 + neg]
                lab = torch.zeros(B, 1 + self.negative, device=self.device)
                lab[:, 0] = 1.0
                out_vecs = self.output[cand]                                       # [B, 1 + neg, dim]
                score = torch.sigmoid((out_vecs * h[:, None, :]).sum(-1))
                gsc = (score - lab)                                                # d loss / d score
                gh = (gsc[:, :, None] * out_vecs).sum(1)
                self._apply(self.output, cand.reshape(-1), -(lr * gsc[:, :, None] * h[:, None, :]).reshape(-1, self.dim))
                self._apply(self.input, idx, -(lr * gh / lens[:, None])[seg])
                seen += B

    # ------------------------------------------------------------------ queries
    def getDimension(self): return self.dim
    def vocab(self): return list(self.words)
    def vocabSize(self): return len(self.words)
    def hasWord(self, w): return w in self.word_index
    def getLabels(self): return [l[len(self.labelPrefix):] for l in self.labels]

    def _vec(self, word):
        rows = self._subwords(word)
        if not rows:
            return torch.zeros(self.dim, device=self.device)
        return self.input[torch.tensor(rows, device=self.device)].mean(0)

    def getWordVector(self, word):
        return self._vec(word).cpu().numpy().astype(np.float64)

    def getWordVectorMatrix(self, word):
        return INDArray(self._vec(word).cpu())

    def similarity(self, a, b):
        va, vb = self._vec(a), self._vec(b)
        d = va.norm() * vb.norm()
        return float((va @ vb) / d) if float(d) > 0 else 0.0

    def wordsNearest(self, word, n=10):
        v = self._vec(word)
        M = torch.stack([self._vec(w) for w in self.words])
        sims = (M @ v) / (M.norm(dim=1) * v.norm() + 1e-12)
        order = torch.argsort(sims, descending=True).tolist()
        return [self.words[i] for i in order if self.words[i] != word][:n]

    def _sentence_probs(self, text):
        if not self.supervised:
            raise RuntimeError("predict needs a supervised model")
        rows = [r for w in text.split() if not w.startswith(self.labelPrefix) for r in self._subwords(w)]
        h, _, _ = self._mean_rows([rows])
        return torch.softmax(h @ self.output.t(), -1)[0]

    def predict(self, text):
        p = self._sentence_probs(text)
        return self.labels[int(torch.argmax(p))][len(self.labelPrefix):]

    def predictProbability(self, text):
        p = self._sentence_probs(text)
        i = int(torch.argmax(p))
        return self.labels[i][len(self.labelPrefix):], float(p[i])

    # ------------------------------------------------------------------ persistence
    def saveModel(self, path):
        meta = {"supervised": self.supervised, "cbow": self.cbow, "dim": self.dim, "minCount": self.minCount, "minn": self.minn,
                "maxn": self.maxn, "bucket": self.bucket, "labelPrefix": self.labelPrefix, "words": self.words, "counts": self.counts,
                "labels": self.labels}
        with zipfile.ZipFile(path, "w", zipfile.ZIP_DEFLATED) as z:
            z.writestr("meta.json", json.dumps(meta))
            for name, t in (("input.npy", self.input), ("output.npy", self.output)):
                buf = io.BytesIO()
                np.save(buf, t.cpu().numpy())
                z.writestr(name, buf.getvalue())

    @staticmethod
    def loadModel(path, device="cpu"):
        with zipfile.ZipFile(path) as z:
            meta = json.loads(z.read("meta.json"))
            ft = FastText(supervised=meta["supervised"], cbow=meta["cbow"], dim=meta["dim"], minCount=meta["minCount"], minn=meta["minn"],
                          maxn=meta["maxn"], bucket=meta["bucket"], labelPrefix=meta["labelPrefix"], device=device)
            ft.words, ft.counts, ft.labels = meta["words"], meta["counts"], meta["labels"]
            ft.word_index = {w: i for i, w in enumerate(ft.words)}
            ft.input = torch.from_numpy(np.load(io.BytesIO(z.read("input.npy")))).to(ft.device)
            ft.output = torch.from_numpy(np.load(io.BytesIO(z.read("output.npy")))).to(ft.device)
        return ft

    loadBinaryModel = loadModel

    def saveVectors(self, path):
        """Text ``.vec`` format: header ``<words> <dim>`` then one word and its vector per line."""
        with open(path, "w", encoding="utf-8") as f:
            f.write(f"{len(self.words)} {self.dim}\n")
            for w in self.words:
                f.write(w + " " + " ".join(f"{x:.5f}" for x in self.getWordVector(w)) + "\n")
