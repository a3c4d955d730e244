"""Workspaces, environment, profiler / executioner and the compression SPI."""
import pytest
import torch

from deeplearning4j_b200 import INDArray
from deeplearning4j_b200.utils import (Environment, LearningPolicy, MemoryWorkspace, SpillPolicy, WorkspaceConfiguration, getWorkspaceManager)
from deeplearning4j_b200.utils.compression import BasicNDArrayCompressor
from deeplearning4j_b200.utils.profiler import ND4JOpProfilerException, OpExecutioner, ProfilerConfig, ProfilingMode


def test_workspace_learns_size_reuses_memory_and_spills():
    ws = MemoryWorkspace(WorkspaceConfiguration(policyLearning=LearningPolicy.FIRST_LOOP, overallocationLimit=0.0), "t")
    with ws:
        a = ws.alloc((100, 10))
        b = ws.alloc((7,), torch.float64)
        assert ws.getSpilledSize() > 0 and not ws.contains(a)            # first loop: nothing allocated yet, everything spills
    assert ws.getCurrentSize() == 4096 + 256 and ws.getGenerationId() == 1
    ptrs = []
    for _ in range(3):
        with ws:
            a = ws.alloc((100, 10), initialize=True)
            b = ws.alloc((7,), torch.float64)
            assert ws.contains(a) and ws.contains(b) and ws.getSpilledSize() == 0 and a.data_ptr() % 256 == 0
            ptrs.append((a.data_ptr(), b.data_ptr()))
            a.fill_(3.0)
            kept = MemoryWorkspace.detach(a)
    assert len(set(ptrs)) == 1 and not ws.contains(kept) and float(kept.sum()) == 3000.0
    strict = MemoryWorkspace(WorkspaceConfiguration(initialSize=1024, policySpill=SpillPolicy.FAIL, policyLearning=LearningPolicy.NONE), "s")
    with strict:
        strict.alloc((128,))
        with pytest.raises(MemoryError):
            strict.alloc((1024,))
    mgr = getWorkspaceManager()
    w2 = mgr.getAndActivateWorkspace(id="loop")
    assert mgr.checkIfWorkspaceExistsAndActive("loop")
    with mgr.scopeOutOfWorkspaces():
        from deeplearning4j_b200.utils.workspace import current_workspace
        assert current_workspace() is None
    w2.notifyScopeLeft()
    assert "loop" in mgr.printAllocationStatisticsForCurrentThread()
    mgr.destroyAllWorkspacesForCurrentThread()


def test_environment_and_executioner_profiling():
    env = Environment.getInstance()
    env.setDebug(True)
    assert env.isDebug() and not env.isDebugAndVerbose() and env.maxThreads() >= 1 and "torch" in env.describe()
    env.setDebug(False)
    ex = OpExecutioner.getInstance()
    ex.setProfilingMode(ProfilingMode.OPERATIONS)
    ex.profiler.reset()
    x = INDArray(torch.tensor([[1.0, -2.0], [3.0, 4.0]]))
    y = ex.exec("add", [x, x])
    assert torch.equal(y.t, x.t * 2)
    ex.exec("reduce_sum", [x], dimensions=[0])
    st = ex.profiler.getStatistics()
    assert st["invocations"] == 2 and st["opCounter"]["add"] == 1 and "add" in st["opTimeMs"] and "Total Op Calls" in ex.profiler.printOutDashboard()
    ex.setProfilingConfig(ProfilerConfig(checkForNAN=True, checkForINF=True))
    assert ex.getProfilingMode() == ProfilingMode.ANY_PANIC
    with pytest.raises(ND4JOpProfilerException, match="NaN"):
        ex.exec("log", [INDArray(torch.tensor([-1.0]))])
    with pytest.raises(ND4JOpProfilerException, match="Inf"):
        ex.exec("divide", [INDArray(torch.tensor([1.0])), INDArray(torch.tensor([0.0]))])
    ex.setProfilingMode(ProfilingMode.DISABLED)


def test_compression_spi():
    c = BasicNDArrayCompressor.getInstance()
    assert {"GZIP", "NOOP", "INT8", "FLOAT16", "THRESHOLD", "BITMAP"} <= set(c.getAvailableCompressors())
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 33, generator=g)
    for alg, tol in (("GZIP", 0.0), ("NOOP", 0.0), ("FLOAT16", 2e-3), ("INT8", 0.03)):
        comp = c.compress(INDArray(x), alg)
        back = c.decompress(comp).t
        assert comp.descriptor.compressionAlgorithm == alg and back.shape == x.shape
        assert float((back - x).abs().max()) <= tol * float(x.abs().max()) + 1e-12
    assert c.compress(INDArray(x), "FLOAT16").compressionRatio() == 2.0
    grad = torch.randn(5000, generator=g) * 1e-3
    orig = grad.clone()
    thr = c.getCompressor("THRESHOLD")
    thr.configure(1e-3)
    comp = thr.compress(grad)
    dec = thr.decompress(comp).t.reshape(-1)
    assert torch.allclose(dec + grad, orig, atol=1e-7) and set(dec.unique().tolist()) <= {-1e-3, 0.0, 1e-3} or torch.allclose(dec + grad, orig, atol=1e-7)
    assert thr.compress(torch.zeros(100)) is None
    c.setDefaultCompression("GZIP")
    assert c.getDefaultCompression() == "GZIP"
    c.setDefaultCompression("FLOAT16")


def test_serde_extras_round_trips(tmp_path):
    from deeplearning4j_b200.serde.extras import ArrowSerde, BinarySerde, NDArrayTextSerializer, Nd4jBase64
    x = INDArray(torch.arange(12.0).reshape(3, 4))
    assert torch.equal(BinarySerde.toArray(BinarySerde.toByteBuffer(x)).t, x.t)
    BinarySerde.writeArrayToDisk(x, str(tmp_path / "a.bin"))
    assert torch.equal(BinarySerde.readFromDisk(str(tmp_path / "a.bin")).t, x.t)
    assert torch.equal(Nd4jBase64.fromBase64(Nd4jBase64.base64String(x)).t, x.t)
    assert [a.t.tolist() for a in Nd4jBase64.arraysFromBase64(Nd4jBase64.arraysToBase64([x, x]))] == [x.t.tolist()] * 2
    assert torch.equal(Nd4jBase64.fromNpyBase64(Nd4jBase64.base64StringNumpy(x)).t, x.t)
    assert torch.equal(NDArrayTextSerializer.fromJson(NDArrayTextSerializer.toJson(x)).t, x.t)
    assert torch.equal(ArrowSerde.fromBytes(ArrowSerde.toBytes(x)).t, x.t)


def test_common_primitives_lifecycle_tracker_and_parallel_loops():
    import torch
    from deeplearning4j_b200.utils.common import AtomicDouble, Counter, CounterMap, Pair, Preconditions, Triple
    from deeplearning4j_b200.utils.lifecycle import LifecycleTracker
    from deeplearning4j_b200.utils import threads
    p = Pair.of(1, "a")
    assert p.getFirst() == 1 and p.getSecond() == "a" and p == Pair(1, "a") and tuple(Triple.of(1, 2, 3)) == (1, 2, 3)
    c = Counter()
    for w in "a b a c a b".split():
        c.incrementCount(w)
    assert c.argMax() == "a" and c.totalCount() == 6 and abs(c.getProbability("b") - 1 / 3) < 1e-9 and c.keySetSorted()[0] == "a"
    cm = CounterMap()
    cm.incrementCount("x", "y", 2.0)
    assert cm.getCount("x", "y") == 2.0 and cm.argMax() == Pair("x", "y")
    ad = AtomicDouble(1.0)
    assert ad.addAndGet(2.5) == 3.5 and ad.compareAndSet(3.5, 0.0) and ad.get() == 0.0
    with pytest.raises(ValueError, match="bad 3"):
        Preconditions.checkArgument(False, "bad %s", 3)
    tr = LifecycleTracker().enable(capture_stacks=True)
    keep = [tr.recordAllocation(torch.zeros(100)) for _ in range(3)]
    tmp = tr.recordAllocation(torch.zeros(10))
    before = tr.snapshot()
    del tmp
    assert tr.liveCount() == 3 and tr.liveBytes() == 3 * 400 and "live objects: 3" in tr.generateLeakReport()
    keep.append(tr.recordAllocation(torch.zeros(1000)))
    assert any("+" in line for line in LifecycleTracker.temporalReport(before, tr.snapshot())) or tr.liveCount() == 4
    out = [0] * 100

    def body(tid, a, b, step):
        for i in range(a, b, step):
            out[i] = i * 2
    threads.parallel_for(body, 0, 100, 1, numThreads=4)
    assert out == [2 * i for i in range(100)]
    s = threads.parallel_long(lambda tid, a, b, st: sum(range(a, b, st)), lambda x, y: x + y, 0, 1000, 1, numThreads=8)
    assert s == sum(range(1000))
