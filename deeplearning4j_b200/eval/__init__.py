"""Evaluation classes (``org/nd4j/evaluation``): classification, binary, calibration, ROC and regression."""
from .classification import ConfusionMatrix, Evaluation, EvaluationAveraging, EvaluationBinary, EvaluationCalibration  # noqa: F401
from .regression import RegressionEvaluation  # noqa: F401
from .roc import ROC, PrecisionRecallCurve, ROCBinary, ROCMultiClass, RocCurve  # noqa: F401
from .tools import EvaluationTools  # noqa: F401
