"""DataSet / MultiDataSet containers, iterators, normalizers and the built-in dataset fetchers
(``nd4j-api/.../linalg/dataset`` and ``deeplearning4j-data``)."""
from .dataset import DataSet, MultiDataSet, SplitTestAndTrain
from .iterators import (AsyncDataSetIterator, AsyncShieldDataSetIterator, BenchmarkDataSetIterator, DataSetIterator,
                        DataSetIteratorSplitter, EarlyTerminationDataSetIterator, ExistingDataSetIterator,
                        INDArrayDataSetIterator, JointParallelDataSetIterator, ListDataSetIterator, MultiDataSetIteratorAdapter,
                        MultiDataSetWrapperIterator, MultipleEpochsIterator, RandomDataSetIterator, SamplingDataSetIterator)
from .normalizers import (CompositeDataSetPreProcessor, DataNormalization, ImagePreProcessingScaler, LabelLastTimeStepPreProcessor,
                          LambdaDataSetPreProcessor, MultiNormalizerMinMaxScaler, MultiNormalizerStandardize, NormalizerMinMaxScaler,
                          NormalizerSerializer, NormalizerStandardize, VGG16ImagePreProcessor)
from .fetchers import (Cifar10DataSetIterator, EmnistDataSetIterator, IrisDataSetIterator, LFWDataSetIterator, MnistDataSetIterator,
                       SvhnDataSetIterator, TinyImageNetDataSetIterator, UciSequenceDataSetIterator)
from .iterators_extra import *  # noqa: F401,F403,E402
