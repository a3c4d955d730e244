"""Model importers: Keras (JSON + weights), TensorFlow frozen GraphDef and ONNX into MultiLayerNetwork / ComputationGraph / SameDiff."""
from .keras_import import (InvalidKerasConfigurationException, KerasModelImport, UnsupportedKerasConfigurationException)  # noqa: F401
from .onnx_import import OnnxFrameworkImporter, importOnnx  # noqa: F401
from .tf_import import TensorflowFrameworkImporter, importFrozenTF  # noqa: F401
from .tflite_import import TFLiteImporter, importTFLite  # noqa: F401
