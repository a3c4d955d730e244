"""Tokenizers, token pre-processors and sentence / document iterators
(``deeplearning4j-nlp/.../text/tokenization``, ``text/sentenceiterator``, ``text/documentiterator``)."""
from __future__ import annotations

import os
import re
import unicodedata


# ----------------------------------------------------------------------------- token pre-processors
class TokenPreProcess:
    def preProcess(self, token): return token


class LowCasePreProcessor(TokenPreProcess):
    def preProcess(self, token): return token.lower()


class CommonPreprocessor(TokenPreProcess):
    """Lower-cases and strips punctuation / digits (``CommonPreprocessor.java``)."""
    _RX = re.compile(r"[\d\.:,\"'\(\)\[\]|/?!;]+")
    def preProcess(self, token): return self._RX.sub("", token).lower()


class EndingPreProcessor(TokenPreProcess):
    def preProcess(self, token):
        for suf in ("s", "ly", "ed", "ing"):
            if token.endswith(suf) and len(token) > len(suf) + 1 and not (suf == "s" and token.endswith("ss")):
                return token[:-len(suf)]
        return token


class StringCleaning:
    @staticmethod
    def stripPunct(s): return re.sub(r"[^\w\s]", "", s)


# ----------------------------------------------------------------------------- tokenizers
class Tokenizer:
    def __init__(self, tokens, pre=None):
        self._tokens = [pre.preProcess(t) for t in tokens] if pre is not None else list(tokens)
        self._tokens = [t for t in self._tokens if t != ""]
        self._i = 0

    def hasMoreTokens(self): return self._i < len(self._tokens)
    def countTokens(self): return len(self._tokens)
    def nextToken(self):
        t = self._tokens[self._i]
        self._i += 1
        return t
    def getTokens(self): return list(self._tokens)
    def setTokenPreProcessor(self, pre):
        self._tokens = [x for x in (pre.preProcess(t) for t in self._tokens) if x != ""]
    def __iter__(self): return iter(self._tokens)


class TokenizerFactory:
    def __init__(self): self.pre = None
    def setTokenPreProcessor(self, pre): self.pre = pre; return self
    def getTokenPreProcessor(self): return self.pre
    def create(self, text): raise NotImplementedError
    def tokenize(self, text): return self.create(text).getTokens()


class DefaultTokenizerFactory(TokenizerFactory):
    """Whitespace tokenizer (``DefaultTokenizer`` wraps ``java.util.StringTokenizer``)."""
    def create(self, text): return Tokenizer(text.split(), self.pre)


class NGramTokenizerFactory(TokenizerFactory):
    def __init__(self, base=None, minN=1, maxN=2):
        super().__init__()
        self.base, self.minN, self.maxN = base or DefaultTokenizerFactory(), minN, maxN

    def create(self, text):
        toks = self.base.create(text).getTokens()
        if self.pre is not None:
            toks = [t for t in (self.pre.preProcess(x) for x in toks) if t]
        out = []
        for n in range(self.minN, self.maxN + 1):
            out += [" ".join(toks[i:i + n]) for i in range(len(toks) - n + 1)]
        return Tokenizer(out)


class BertWordPiecePreProcessor(TokenPreProcess):
    """Text clean-up applied before word-piece splitting: optional lower-casing + accent stripping, control characters
    removed, whitespace normalised (``BertWordPiecePreProcessor.java``)."""

    def __init__(self, lowerCase=False, stripAccents=False, vocab=None):
        self.lowerCase, self.stripAccents, self.vocab = lowerCase, stripAccents, vocab

    def preProcess(self, text):
        if self.lowerCase:
            text = text.lower()
        if self.stripAccents:
            text = "".join(c for c in unicodedata.normalize("NFD", text) if unicodedata.category(c) != "Mn")
        out = []
        for c in text:
            cp = ord(c)
            if cp == 0 or cp == 0xFFFD or (unicodedata.category(c) in ("Cc", "Cf") and c not in "\t\n\r"):
                continue
            out.append(" " if c.isspace() else c)
        return "".join(out)


def _is_punct(c):
    cp = ord(c)
    if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
        return True
    return unicodedata.category(c).startswith("P")


def _is_cjk(cp):
    return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF or 0x2A700 <= cp <= 0x2B73F or
            0x2B740 <= cp <= 0x2B81F or 0x2B820 <= cp <= 0x2CEAF or 0xF900 <= cp <= 0xFAFF or 0x2F800 <= cp <= 0x2FA1F)


class BertWordPieceTokenizerFactory(TokenizerFactory):
    """Greedy longest-match-first word-piece tokenizer over a BERT vocabulary (``BertWordPieceTokenizer.java``):
    split on whitespace and punctuation (CJK characters become their own tokens), then split every word into the
    longest vocabulary pieces, continuation pieces prefixed with ``##``; unknown words become ``[UNK]``."""

    def __init__(self, vocab, lowerCaseOnly=False, stripAccents=False, charset="utf-8", maxCharsPerWord=100, unk="[UNK]"):
        super().__init__()
        if isinstance(vocab, (str, os.PathLike)):
            with open(vocab, encoding=charset) as f:
                vocab = [l.rstrip("\n") for l in f]
        if isinstance(vocab, (list, tuple)):
            vocab = {t: i for i, t in enumerate(vocab)}
        self.vocab = dict(vocab)
        self.inv = {i: t for t, i in self.vocab.items()}
        self.unk, self.maxChars = unk, maxCharsPerWord
        self.pre = BertWordPiecePreProcessor(lowerCaseOnly, stripAccents, self.vocab)

    def getVocab(self): return self.vocab

    def _basic(self, text):
        out, cur = [], []
        for c in text:
            if c.isspace():
                if cur:
                    out.append("".join(cur)); cur = []
            elif _is_punct(c) or _is_cjk(ord(c)):
                if cur:
                    out.append("".join(cur)); cur = []
                out.append(c)
            else:
                cur.append(c)
        if cur:
            out.append("".join(cur))
        return out

    def _wordpiece(self, word):
        if len(word) > self.maxChars:
            return [self.unk]
        pieces, start = [], 0
        while start < len(word):
            end, cur = len(word), None
            while start < end:
                sub = word[start:end]
                if start > 0:
                    sub = "##" + sub
                if sub in self.vocab:
                    cur = sub
                    break
                end -= 1
            if cur is None:
                return [self.unk]
            pieces.append(cur)
            start = end
        return pieces

    def create(self, text):
        text = self.pre.preProcess(text) if self.pre is not None else text
        toks = []
        for w in self._basic(text):
            toks.extend(self._wordpiece(w))
        return Tokenizer(toks)

    def encode(self, text): return [self.vocab.get(t, self.vocab.get(self.unk, 0)) for t in self.create(text).getTokens()]
    def decode(self, ids):
        out = []
        for i in ids:
            t = self.inv.get(int(i), self.unk)
            if t.startswith("##") and out:
                out[-1] += t[2:]
            else:
                out.append(t)
        return " ".join(out)


# ----------------------------------------------------------------------------- sentence / document iterators
class SentenceIterator:
    def __init__(self): self.preProcessor = None
    def setPreProcessor(self, p): self.preProcessor = p
    def getPreProcessor(self): return self.preProcessor
    def _pp(self, s): return self.preProcessor(s) if callable(self.preProcessor) else (self.preProcessor.preProcess(s) if self.preProcessor else s)
    def __iter__(self):
        self.reset()
        while self.hasNext():
            yield self.nextSentence()


class CollectionSentenceIterator(SentenceIterator):
    def __init__(self, coll):
        super().__init__()
        self.coll, self.i = list(coll), 0
    def hasNext(self): return self.i < len(self.coll)
    def nextSentence(self):
        s = self.coll[self.i]
        self.i += 1
        return self._pp(s)
    def reset(self): self.i = 0
    def finish(self): pass


class BasicLineIterator(SentenceIterator):
    """One sentence per line of a text file."""
    def __init__(self, path, encoding="utf-8"):
        super().__init__()
        self.path, self.encoding, self.f, self._next = str(path), encoding, None, None
        self.reset()
    def reset(self):
        if self.f:
            self.f.close()
        self.f = open(self.path, encoding=self.encoding)
        self._advance()
    def _advance(self):
        line = self.f.readline()
        self._next = None if line == "" else line.rstrip("\n")
    def hasNext(self): return self._next is not None
    def nextSentence(self):
        s = self._next
        self._advance()
        return self._pp(s)
    def finish(self):
        if self.f:
            self.f.close()
            self.f = None

LineSentenceIterator = BasicLineIterator


class FileSentenceIterator(SentenceIterator):
    """Every line of every file under a directory."""
    def __init__(self, directory):
        super().__init__()
        self.files = sorted(os.path.join(r, f) for r, _, fs in os.walk(str(directory)) for f in fs) if os.path.isdir(str(directory)) else [str(directory)]
        self.reset()
    def reset(self):
        self.lines = (line.rstrip("\n") for p in self.files for line in open(p, encoding="utf-8", errors="ignore"))
        self._next = next(self.lines, None)
    def hasNext(self): return self._next is not None
    def nextSentence(self):
        s = self._next
        self._next = next(self.lines, None)
        return self._pp(s)
    def finish(self): pass


class LabelledDocument:
    def __init__(self, content="", labels=None, id=None):
        self.content, self.labels, self.id = content, list(labels or []), id
        self.referencedContent = None
    def getContent(self): return self.content
    def getLabels(self): return self.labels
    def getLabel(self): return self.labels[0] if self.labels else None
    def addLabel(self, l): self.labels.append(l)


class LabelsSource:
    def __init__(self, template_or_labels="DOC_"):
        self.template = template_or_labels if isinstance(template_or_labels, str) else None
        self.labels = [] if self.template else list(template_or_labels)
        self.counter = 0
    def nextLabel(self):
        l = f"{self.template}{self.counter}"
        self.counter += 1
        self.labels.append(l)
        return l
    def storeLabel(self, l):
        if l not in self.labels:
            self.labels.append(l)
    def getLabels(self): return list(self.labels)
    def reset(self): self.counter = 0


class LabelAwareIterator:
    def __iter__(self):
        self.reset()
        while self.hasNextDocument():
            yield self.nextDocument()


class SimpleLabelAwareIterator(LabelAwareIterator):
    def __init__(self, docs):
        self.docs, self.i = list(docs), 0
        self.source = LabelsSource([l for d in self.docs for l in d.getLabels()])
    def hasNextDocument(self): return self.i < len(self.docs)
    def nextDocument(self):
        d = self.docs[self.i]
        self.i += 1
        return d
    def reset(self): self.i = 0
    def getLabelsSource(self): return self.source


class SentenceIteratorConverter(LabelAwareIterator):
    """Wraps a SentenceIterator, labelling sentence ``i`` as ``DOC_i``."""
    def __init__(self, it, source=None):
        self.it, self.source = it, source or LabelsSource("DOC_")
    def hasNextDocument(self): return self.it.hasNext()
    def nextDocument(self): return LabelledDocument(self.it.nextSentence(), [self.source.nextLabel()])
    def reset(self):
        self.it.reset()
        self.source.reset()
    def getLabelsSource(self): return self.source


class FileLabelAwareIterator(LabelAwareIterator):
    """Sub-directory name = label, each file = one document."""
    def __init__(self, root):
        self.items = []
        for lab in sorted(os.listdir(str(root))):
            d = os.path.join(str(root), lab)
            if os.path.isdir(d):
                self.items += [(os.path.join(d, f), lab) for f in sorted(os.listdir(d))]
        self.source = LabelsSource(sorted({l for _, l in self.items}))
        self.i = 0

    class Builder:
        def __init__(self): self.root = None
        def addSourceFolder(self, p): self.root = p; return self
        def build(self): return FileLabelAwareIterator(self.root)

    def hasNextDocument(self): return self.i < len(self.items)
    def nextDocument(self):
        p, lab = self.items[self.i]
        self.i += 1
        return LabelledDocument(open(p, encoding="utf-8", errors="ignore").read(), [lab])
    def reset(self): self.i = 0
    def getLabelsSource(self): return self.source
