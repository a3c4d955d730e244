"""Tokenizers, Word2Vec / ParagraphVectors training and serialisation, BertIterator."""
import numpy as np
import random

import torch

from deeplearning4j_b200.nlp import (BertIterator, BertMaskedLMMasker, BertWordPieceTokenizerFactory, CollectionLabeledSentenceProvider,
                                     CollectionSentenceIterator, CommonPreprocessor, DefaultTokenizerFactory, LabelledDocument,
                                     NGramTokenizerFactory, ParagraphVectors, VocabCache, Word2Vec, WordVectorSerializer, build_huffman)


def _corpus(n=400, seed=0):
    r = random.Random(seed)
    animals, foods = ["cat", "dog", "horse", "cow"], ["bread", "cheese", "apple", "rice"]
    out = []
    for _ in range(n):
        if r.random() < 0.5:
            out.append(" ".join(["the"] + [r.choice(animals) for _ in range(6)] + ["runs"]))
        else:
            out.append(" ".join(["we"] + [r.choice(foods) for _ in range(6)] + ["eat"]))
    return out


def test_tokenizers():
    tf = DefaultTokenizerFactory().setTokenPreProcessor(CommonPreprocessor())
    assert tf.create("Hello, World! 42 times.").getTokens() == ["hello", "world", "times"]
    assert NGramTokenizerFactory(DefaultTokenizerFactory(), 1, 2).create("a b c").getTokens() == ["a", "b", "c", "a b", "b c"]
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "un", "##aff", "##able", "the", "cat", ",", "##s", "é"]
    wp = BertWordPieceTokenizerFactory(vocab, lowerCaseOnly=True, stripAccents=True)
    assert wp.create("The unaffable cats, xyz").getTokens() == ["the", "un", "##aff", "##able", "cat", "##s", ",", "[UNK]"]
    assert wp.decode(wp.encode("unaffable cats")) == "unaffable cats"


def test_huffman_codes_are_prefix_free_and_frequency_ordered():
    vc = VocabCache()
    for w, c in [("a", 50), ("b", 20), ("c", 10), ("d", 5), ("e", 1)]:
        vc.incrementWordCount(w, c)
    vc.finalize_(1)
    inner = build_huffman(vc)
    codes = ["".join(map(str, v.codes)) for v in vc.by_index]
    assert inner == 4 and len(codes[0]) <= len(codes[-1])
    assert not any(a != b and b.startswith(a) for a in codes for b in codes)
    assert all(0 <= p < inner for v in vc.by_index for p in v.points)


def _cluster_score(vec):
    same = (vec.similarity("cat", "dog") + vec.similarity("bread", "cheese")) / 2
    diff = (vec.similarity("cat", "bread") + vec.similarity("dog", "rice")) / 2
    return same - diff


def test_word2vec_skipgram_negative_sampling_and_hs_learn_clusters(tmp_path):
    for kw in (dict(negativeSample=5, useHierarchicSoftmax=False), dict(negativeSample=0, useHierarchicSoftmax=True),
               dict(negativeSample=5, useHierarchicSoftmax=False, elementsLearningAlgorithm="CBOW")):
        vec = (Word2Vec.Builder().minWordFrequency(1).layerSize(24).windowSize(3).epochs(12).seed(7).batchSize(256).learningRate(0.05)
               .iterate(CollectionSentenceIterator(_corpus())).tokenizerFactory(DefaultTokenizerFactory()).device("cpu").build())
        for k, v in kw.items():
            setattr(vec, k, v)
        vec.fit()
        assert _cluster_score(vec) > 0.3, (kw, _cluster_score(vec))
        assert set(vec.wordsNearest("cat", 3)) <= {"dog", "horse", "cow", "the", "runs"}
    p = str(tmp_path / "w2v.zip")
    WordVectorSerializer.writeWord2VecModel(vec, p)
    back = WordVectorSerializer.readWord2VecModel(p)
    assert back.vocab.words_() == vec.vocab.words_() and torch.allclose(back.lookupTable.syn0, vec.lookupTable.syn0, atol=1e-6)
    WordVectorSerializer.writeWordVectors(vec, str(tmp_path / "v.txt"))
    txt = WordVectorSerializer.loadTxtVectors(str(tmp_path / "v.txt"))
    assert abs(txt.similarity("cat", "dog") - vec.similarity("cat", "dog")) < 1e-4
    WordVectorSerializer.writeBinary(vec, str(tmp_path / "v.bin"))
    b = WordVectorSerializer.readBinaryModel(str(tmp_path / "v.bin"))
    assert torch.allclose(b.lookupTable.syn0, vec.lookupTable.syn0.cpu())
    assert vec.getWordVectorMatrix("cat").t.shape == (24,) and vec.getWordVector("nonexistent") is None


def test_paragraph_vectors_labels_and_inference():
    docs = [LabelledDocument(s, ["ANIMAL" if s.startswith("the") else "FOOD"]) for s in _corpus(300, 1)]
    pv = (ParagraphVectors.Builder().minWordFrequency(1).layerSize(20).windowSize(3).epochs(10).seed(3).batchSize(256).learningRate(0.05)
          .negativeSample(5).useHierarchicSoftmax(False).iterate(docs).device("cpu").build())
    pv.fit()
    assert pv.predict("the cat dog cow runs") == "ANIMAL" and pv.predict("we bread apple rice eat") == "FOOD"
    assert pv.nearestLabels("the horse horse runs", 2)[0] == "ANIMAL"
    assert pv.similarityToLabel("we cheese cheese eat", "FOOD") > pv.similarityToLabel("we cheese cheese eat", "ANIMAL")
    assert pv.inferVector("the cat runs").t.shape == (20,)


def test_bert_iterator_unsupervised_and_classification():
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"] + [f"w{i}" for i in range(50)]
    tf = BertWordPieceTokenizerFactory(vocab)
    sents = [" ".join(f"w{(i * 7 + j) % 50}" for j in range(5 + i % 9)) for i in range(20)]
    it = (BertIterator.builder().tokenizer(tf).lengthHandling(BertIterator.LengthHandling.FIXED_LENGTH, 12).minibatchSize(8)
          .sentenceProvider(CollectionLabeledSentenceProvider(sents, ["a"] * 20)).featureArrays(BertIterator.FeatureArrays.INDICES_MASK)
          .vocabMap(tf.getVocab()).task(BertIterator.Task.UNSUPERVISED).masker(BertMaskedLMMasker(random.Random(1), 0.3, 0.8, 0.1))
          .unsupervisedLabelFormat(BertIterator.UnsupervisedLabelFormat.RANK2_IDX).build())
    batches = list(it)
    assert [b.getFeatures(0).shape[0] for b in batches] == [8, 8, 4]
    b = batches[0]
    idx, fmask, lab, lmask = b.getFeatures(0), b.getFeaturesMaskArray(0), b.getLabels(0), b.getLabelsMaskArray(0)
    assert idx.shape == (8, 12) and bool((idx[:, 0] == 2).all()) and float(lmask[:, 0].sum()) == 0
    changed = (idx != lab) & (fmask > 0)
    assert bool(((lmask > 0) | ~changed).all()) and 0 < float(lmask.sum()) < float(fmask.sum())
    assert bool((idx[changed] == 4).float().mean() > 0.5)
    cls = (BertIterator.builder().tokenizer(tf).lengthHandling(BertIterator.LengthHandling.CLIP_ONLY, 8).minibatchSize(5)
           .sentenceProvider(CollectionLabeledSentenceProvider(sents, ["pos" if i % 2 else "neg" for i in range(20)]))
           .featureArrays(BertIterator.FeatureArrays.INDICES_MASK_SEGMENTID).vocabMap(tf.getVocab())
           .task(BertIterator.Task.SEQ_CLASSIFICATION).build())
    m = cls.next()
    assert m.getFeatures(0).shape[1] <= 8 and m.getLabels(0).shape == (5, 2) and len(m.getFeatures()) == 2
    assert float(m.getLabels(0).sum()) == 5.0
    feats, masks = cls.featurizeSentencePairs([("w1 w2 w3", "w4 w5")])
    assert feats[1][0].tolist()[:7] == [0, 0, 0, 0, 0, 1, 1]


def test_fasttext_supervised_and_subword_vectors(tmp_path):
    from deeplearning4j_b200.nlp.fasttext import FastText
    rng = np.random.default_rng(0)
    animals = "cat dog horse cow sheep goat tiger lion".split()
    tools = "hammer wrench drill saw pliers chisel ruler level".split()
    lines = []
    for _ in range(300):
        if rng.random() < 0.5:
            lines.append("__label__animal " + " ".join(rng.choice(animals, 5)))
        else:
            lines.append("__label__tool " + " ".join(rng.choice(tools, 5)))
    ft = FastText(supervised=True, dim=16, epochs=20, lr=0.5, minn=2, maxn=4, bucket=2000, iterator=lines, batchSize=64, seed=1).fit()
    assert set(ft.getLabels()) == {"animal", "tool"}
    assert ft.predict("the cat and the lion") == "animal" and ft.predict("wrench drill saw") == "tool"
    lab, p = ft.predictProbability("hammer chisel")
    assert lab == "tool" and 0.5 < p <= 1.0
    # an unseen word still gets a vector from its character n-grams, close to a word it shares most n-grams with
    assert not ft.hasWord("hammers") and np.abs(ft.getWordVector("hammers")).sum() > 0
    path = str(tmp_path / "ft.zip")
    ft.saveModel(path)
    back = FastText.loadModel(path)
    assert back.predict("goat sheep cow") == "animal"
    np.testing.assert_allclose(back.getWordVector("cat"), ft.getWordVector("cat"))
    # skip-gram mode trains word + sub-word vectors; words that share contexts end up closer than unrelated ones
    corpus = [" ".join(rng.choice(animals, 8)) for _ in range(200)] + [" ".join(rng.choice(tools, 8)) for _ in range(200)]
    sg = FastText(skipgram=True, dim=24, epochs=8, lr=0.1, minn=0, maxn=0, iterator=corpus, batchSize=512, negativeSamples=5, seed=3).fit()
    assert sg.similarity("cat", "dog") > sg.similarity("cat", "wrench")
    assert len(sg.wordsNearest("hammer", 3)) == 3
