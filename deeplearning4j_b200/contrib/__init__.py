"""Developer tools that ship with the framework (the reference's ``contrib/`` tree): an op-execution log with regression diffing
(``nd4j-log-analyzer``) and a profile summariser (``unified-profiler-analyzer``)."""
from .op_log import OpLogAnalyzer, OpLogListener  # noqa: F401
