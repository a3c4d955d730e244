"""The native workspace arena on host memory (the device kind runs in the GPU tests)."""
import pytest
import torch

from deeplearning4j_b200.utils.arena import DEVICE, HOST, NativeArena


def test_bump_allocation_spill_learning_and_resize():
    a = NativeArena(HOST, 4096)
    x = a.tensor((8, 16), torch.float32, zero=True)             # 512 B
    y = a.tensor((100,), torch.float64)                          # 800 B -> 1024 with the 256-byte granule
    assert x.data_ptr() % 256 == 0 and y.data_ptr() % 256 == 0 and y.data_ptr() - x.data_ptr() == 512
    x.fill_(3.0)
    y.fill_(-1.0)
    assert float(x.sum()) == 3.0 * 128 and float(y.sum()) == -100.0          # no overlap
    st = a.stats()
    assert st["capacity"] == 4096 and st["offset"] == 512 + 1024 and st["spillBlocks"] == 0
    big = a.tensor((2000,), torch.float32)                       # 8000 B: does not fit -> spill block
    big.zero_()
    st = a.stats()
    assert st["spillBlocks"] == 1 and st["spilledBytes"] >= 8000 and st["offset"] == 1536
    with pytest.raises(MemoryError):
        a.tensor((2000,), torch.float32, allowSpill=False)
    with pytest.raises(RuntimeError, match="between cycles"):
        a.resize(1 << 16)
    a.reset()
    st = a.stats()
    assert st["offset"] == 0 and st["spillBlocks"] == 0 and st["generation"] == 1 and st["maxCycleBytes"] >= 512 + 1024 + 8000
    a.resize(st["maxCycleBytes"] * 2)                            # the learned size: the next cycle fits without spilling
    for _ in range(3):
        a.tensor((8, 16)); a.tensor((100,), torch.float64); a.tensor((2000,))
        assert a.stats()["spillBlocks"] == 0
        a.reset()
    z = a.tensor((4,), torch.bfloat16, zero=True)
    assert z.dtype == torch.bfloat16 and z.tolist() == [0, 0, 0, 0]
    e = a.tensor((0, 3))
    assert tuple(e.shape) == (0, 3)
    a.close()


@pytest.mark.gpu
def test_device_arena_tensors():
    a = NativeArena(DEVICE, 1 << 20)
    x = a.tensor((256, 256), torch.float32, zero=True)
    y = a.tensor((1000,), torch.bfloat16, zero=True)
    assert x.is_cuda and y.is_cuda and x.data_ptr() % 256 == 0
    x += 1
    y += 2
    torch.cuda.synchronize()
    assert float(x.sum()) == 65536 and float(y.float().sum()) == 2000
    assert a.stats()["offset"] == 256 * 256 * 4 + 2048
    a.reset()
    a.close()


def test_workspace_over_the_native_arena_follows_the_same_policies():
    from deeplearning4j_b200.utils.workspace import (BasicWorkspaceManager, LearningPolicy, MemoryWorkspace, NativeMemoryWorkspace, SpillPolicy,
                                                     WorkspaceConfiguration)
    conf = WorkspaceConfiguration.builder().policyLearning(LearningPolicy.FIRST_LOOP).overallocationLimit(0.5).build()
    mgr = BasicWorkspaceManager()
    ws = mgr.createNewWorkspace(conf, "nat", native=True)
    ref = MemoryWorkspace(conf, "ref")
    assert isinstance(ws, NativeMemoryWorkspace)
    for w in (ws, ref):
        with w:
            a = w.alloc((10, 10), torch.float32, True)
            b = w.alloc((7,), torch.float64, False)
            a += 1
            assert float(a.sum()) == 100.0 and tuple(b.shape) == (7,)
            assert w.getSpilledSize() > 0                          # first cycle: nothing learned yet, everything spills
        assert w.getCurrentSize() >= int((512 + 256) * 1.5) // 256 * 256 and w.getGenerationId() == 1
        with w:
            w.alloc((10, 10), torch.float32)
            w.alloc((7,), torch.float64)
            assert w.getSpilledSize() == 0 and w.getCurrentOffset() == 768
    assert ws.getCurrentSize() == ref.getCurrentSize()
    strict = NativeMemoryWorkspace(WorkspaceConfiguration.builder().initialSize(1024).policySpill(SpillPolicy.FAIL).build(), "strict")
    with strict:
        strict.alloc((128,), torch.float32)
        with pytest.raises(MemoryError):
            strict.alloc((1024,), torch.float32)
    ws.destroyWorkspace()
    assert ws.getCurrentSize() == 0
