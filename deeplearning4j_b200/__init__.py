"""deeplearning4j_b200 — a Blackwell-native deep-learning framework with Deeplearning4j's
capabilities, API shape and checkpoint formats (ND4J arrays/ops, SameDiff graphs,
MultiLayerNetwork / ComputationGraph, ModelSerializer zips, ParallelWrapper gradient sharing)
on top of PyTorch tensors and hand-written sm_100a CUDA kernels."""
__version__ = "0.1.0"

from .nd.dtype import DataType
from .nd.ndarray import INDArray, NDArrayIndex
from .nd.nd4j import Nd4j, Transforms
