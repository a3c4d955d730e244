"""SameDiff: define-then-run graphs with autodiff, training and the FlatBuffers / SDNB / SDZ save formats
(``nd4j-api/.../autodiff/samediff/SameDiff.java``)."""
from .core import SameDiff, SDVariable, SameDiffOp, VariableType
from .training import History, TrainingConfig

__all__ = ["SameDiff", "SDVariable", "SameDiffOp", "VariableType", "TrainingConfig", "History"]
