"""Runtime environment flags (``libnd4j/include/system/Environment.h:43-122`` and the Java side
``ND4JSystemProperties`` / ``ND4JEnvironmentVars``).  One process-wide ``Environment`` whose fields are seeded
from environment variables and can be changed at run time; the native library reads none of them itself,
they steer the Python runtime (profiling, verbosity, thread caps, kernel selection)."""
from __future__ import annotations

import os
import threading


class ND4JEnvironmentVars:
    BACKEND_PRIORITY_CPU = "BACKEND_PRIORITY_CPU"
    BACKEND_PRIORITY_GPU = "BACKEND_PRIORITY_GPU"
    OMP_NUM_THREADS = "OMP_NUM_THREADS"
    SD_MAX_THREADS = "SD_MAX_THREADS"
    ND4J_RESOURCES_CACHE_DIR = "ND4J_RESOURCES_CACHE_DIR"
    ND4J_TEST_RESOURCES = "ND4J_TEST_RESOURCES"
    ND4J_SKIP_BLAS_THREADS = "ND4J_SKIP_BLAS_THREADS"
    # this framework's own switches
    DL4J_B200_FORCE_TORCH = "DL4J_B200_FORCE_TORCH"      # 1: never dispatch to the native kernels
    DL4J_B200_DEBUG = "DL4J_B200_DEBUG"
    DL4J_B200_VERBOSE = "DL4J_B200_VERBOSE"
    DL4J_B200_PROFILING = "DL4J_B200_PROFILING"


class ND4JSystemProperties:
    DTYPE = "dtype"
    LOG_INITIALIZATION = "org.nd4j.log.initialization"
    RESOURCES_CACHE_DIR = "org.nd4j.test.resources.cache.dir"
    WORKSPACE_DEBUG = "org.nd4j.workspace.debug"
    VERSION_CHECK = "org.nd4j.versioncheck"


def _flag(name, default=False):
    v = os.environ.get(name)
    return default if v is None else v.strip().lower() in ("1", "true", "yes", "on")


class Environment:
    _instance = None
    _lock = threading.Lock()

    def __init__(self):
        E = ND4JEnvironmentVars
        self._debug = _flag(E.DL4J_B200_DEBUG)
        self._verbose = _flag(E.DL4J_B200_VERBOSE)
        self._profiling = _flag(E.DL4J_B200_PROFILING)
        self._detect_leaks = False
        self._helpers_allowed = not _flag(E.DL4J_B200_FORCE_TORCH)
        self._max_threads = int(os.environ.get(E.SD_MAX_THREADS, os.environ.get(E.OMP_NUM_THREADS, os.cpu_count() or 1)))
        self._max_master_threads = self._max_threads
        self._tad_threshold = 8
        self._elementwise_threshold = 32768
        self._max_primary_memory = 0
        self._max_special_memory = 0
        self._max_device_memory = 0
        self._precision_boost = False
        self._experimental = False
        self._default_float = "FLOAT"
        self._delete_shape_info = True
        self._delete_primary = True
        self._delete_special = True
        self._last_error = (0, "")
        self.variables = {}

    @classmethod
    def getInstance(cls):
        with cls._lock:
            if cls._instance is None:
                cls._instance = cls()
            return cls._instance

    # flags -------------------------------------------------------------
    def isDebug(self): return self._debug
    def setDebug(self, b): self._debug = bool(b)
    def isVerbose(self): return self._verbose
    def setVerbose(self, b): self._verbose = bool(b)
    def isProfiling(self): return self._profiling
    def setProfiling(self, b): self._profiling = bool(b)
    def isDetectingLeaks(self): return self._detect_leaks
    def setLeaksDetector(self, b): self._detect_leaks = bool(b)
    def isDebugAndVerbose(self): return self._debug and self._verbose
    def isExperimentalBuild(self): return self._experimental
    def precisionBoostAllowed(self): return self._precision_boost
    def allowPrecisionBoost(self, b): self._precision_boost = bool(b)

    def helpersAllowed(self): return self._helpers_allowed

    def allowHelpers(self, b):
        """Native-kernel dispatch on/off (the reference toggles cuDNN / oneDNN helpers with this flag)."""
        self._helpers_allowed = bool(b)
        from ..ops import nnops
        nnops.set_force_torch(not self._helpers_allowed)

    # sizes -------------------------------------------------------------
    def maxThreads(self): return self._max_threads
    def setMaxThreads(self, n):
        import torch
        self._max_threads = max(int(n), 1)
        torch.set_num_threads(self._max_threads)
    def maxMasterThreads(self): return self._max_master_threads
    def setMaxMasterThreads(self, n): self._max_master_threads = max(int(n), 1)
    def tadThreshold(self): return self._tad_threshold
    def setTadThreshold(self, n): self._tad_threshold = int(n)
    def elementwiseThreshold(self): return self._elementwise_threshold
    def setElementwiseThreshold(self, n): self._elementwise_threshold = int(n)
    def setMaxPrimaryMemory(self, n): self._max_primary_memory = int(n)
    def setMaxSpecialMemory(self, n): self._max_special_memory = int(n)
    def setMaxDeviceMemory(self, n):
        import torch
        self._max_device_memory = int(n)
        if n and torch.cuda.is_available():
            total = torch.cuda.get_device_properties(0).total_memory
            torch.cuda.set_per_process_memory_fraction(min(1.0, n / total))
    def maxPrimaryMemory(self): return self._max_primary_memory
    def maxSpecialMemory(self): return self._max_special_memory
    def maxDeviceMemory(self): return self._max_device_memory
    def defaultFloatDataType(self): return self._default_float
    def setDefaultFloatDataType(self, dt): self._default_float = getattr(dt, "name", str(dt))

    # device ------------------------------------------------------------
    def isCPU(self):
        import torch
        return not torch.cuda.is_available()

    def blasMajorVersion(self):
        import torch
        return int((torch.version.cuda or "0.0").split(".")[0])

    def blasMinorVersion(self):
        import torch
        return int((torch.version.cuda or "0.0").split(".")[1])

    def capabilities(self):
        import torch
        return [torch.cuda.get_device_capability(i) for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else []

    # errors ------------------------------------------------------------
    def lastErrorCode(self): return self._last_error[0]
    def lastErrorMessage(self): return self._last_error[1]
    def setLastError(self, code, message): self._last_error = (int(code), str(message))

    def describe(self):
        import torch
        return {"debug": self._debug, "verbose": self._verbose, "profiling": self._profiling, "helpersAllowed": self._helpers_allowed,
                "maxThreads": self._max_threads, "cuda": torch.version.cuda, "devices": torch.cuda.device_count() if torch.cuda.is_available() else 0,
                "torch": torch.__version__}
