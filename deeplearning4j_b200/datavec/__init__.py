"""DataVec: record readers / writers, input splits, Schema + TransformProcess, DataSet iterators over records."""
from .records import *  # noqa: F401,F403
from .records import (AlignmentMode, RecordReaderDataSetIterator, SequenceRecordReaderDataSetIterator)  # noqa: F401
from .transform import (AnalyzeLocal, BooleanCondition, CategoricalColumnCondition, ColumnCondition, ColumnType, ConditionFilter,  # noqa: F401
                        ConditionOp, DataAnalysis, DoubleColumnCondition, IntegerColumnCondition, InvalidValueColumnCondition,
                        LocalTransformExecutor, MathFunction, MathOp, NullWritableColumnCondition, ReduceOp, Reducer, Schema,
                        StringColumnCondition, TransformProcess)
