"""DataVec: record readers / writers, input splits, Schema + TransformProcess, DataSet iterators over records."""
from .records import *  # noqa: F401,F403
from .records import (AlignmentMode, RecordReaderDataSetIterator, SequenceRecordReaderDataSetIterator)  # noqa: F401
from .transform import (AnalyzeLocal, BooleanCondition, CategoricalColumnCondition, ColumnCondition, ColumnType, ConditionFilter,  # noqa: F401
                        ConditionOp, DataAnalysis, DoubleColumnCondition, IntegerColumnCondition, InvalidValueColumnCondition,
                        LocalTransformExecutor, MathFunction, MathOp, NullWritableColumnCondition, ReduceOp, Reducer, Schema,
                        StringColumnCondition, TransformProcess, Distance, OverlappingTimeWindowFunction, SequenceSplitTimeSeparation,
                        SplitMaxLengthSequence, TimeWindowFunction)
from .extra import (ArrowConverter, ArrowRecordReader, ArrowRecordWriter, BoxImageTransform, ColorConversionTransform,  # noqa: F401
                    CropImageTransform, DataQualityAnalysis, EqualizeHistTransform, ExcelRecordReader, ExcelRecordWriter,
                    FlipImageTransform, ImageTransform, JDBCRecordReader, Join, JoinType, MultiImageTransform, NativeImageLoader,
                    PipelineImageTransform, RandomCropTransform, ResizeImageTransform, RotateImageTransform, ScaleImageTransform,
                    analyzeQuality, convertFromSequence, executeJoin, reduceSequence, sequenceDifference,
                    sequenceMovingWindowReduce, splitSequenceMaxLength, splitSequenceTimeSeparation, trimSequence,
                    trimSequenceToLength)

LocalTransformExecutor.executeJoin = staticmethod(executeJoin)
AnalyzeLocal.analyzeQuality = staticmethod(analyzeQuality)
