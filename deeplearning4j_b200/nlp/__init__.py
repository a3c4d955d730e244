"""NLP: tokenizers, sentence / document iterators, Word2Vec, ParagraphVectors, BERT data pipeline."""
from .bert_iterator import (BertIterator, BertMaskedLMMasker, CollectionLabeledPairSentenceProvider,  # noqa: F401
                            CollectionLabeledSentenceProvider)
from .embeddings import (InMemoryLookupTable, ParagraphVectors, SequenceVectors, VocabCache, VocabWord, Word2Vec,  # noqa: F401
                         WordVectorSerializer, build_huffman)
from .tokenization import *  # noqa: F401,F403
from .fasttext import FastText  # noqa: F401
