"""DistributedINDArray on two gloo ranks (CPU): allocation, propagate, entry(i) of a peer, sync of a SYNCABLE array."""
import os
import sys

import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deeplearning4j_b200 import DataType
    from deeplearning4j_b200.nd.distributed import ArrayType, DistributedINDArray
    d = DistributedINDArray(ArrayType.SYNCABLE, device="cpu").allocateAll(DataType.FLOAT, 3, 4)
    assert d.numEntries() == world and d.numActiveEntries() == world and d.getINDArrayType() is ArrayType.SYNCABLE
    d.entry().t.fill_(float(rank + 1))
    peer = d.entry(1)                                   # collective: everybody asks for entry 1
    assert torch.equal(peer.t, torch.full((3, 4), 2.0))
    d.sync(mean=True)
    assert torch.allclose(d.entry().t, torch.full((3, 4), (1 + world) / 2))
    c = DistributedINDArray(ArrayType.CONSTANT, device="cpu")
    c.propagate(torch.arange(6.0).reshape(2, 3) if rank == 0 else None, src=0)
    assert torch.equal(c.entry().t, torch.arange(6.0).reshape(2, 3))
    v = DistributedINDArray(ArrayType.VARIADIC, device="cpu")
    for e in range(world):
        v.allocate(e, DataType.INT, e + 1)
    assert tuple(v.entry().t.shape) == (rank + 1,)
    v.entry().t.fill_(7 + rank)
    assert torch.equal(v.entry(0).t, torch.full((1,), 7, dtype=torch.int32))
    try:
        v.sync()
        raise AssertionError("sync of a VARIADIC array must raise")
    except ValueError:
        pass
    try:
        DistributedINDArray(ArrayType.CONSTANT, device="cpu").allocate(0, DataType.FLOAT, 2).allocate(1, DataType.FLOAT, 3)
        raise AssertionError("CONSTANT entries of different shapes must raise")
    except ValueError:
        pass
    dist.barrier()
    torch.save({"ok": True}, os.path.join(out, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_distributed_ndarray_two_ranks(tmp_path):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, 29641, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive() and p.exitcode == 0
    assert all(os.path.exists(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(2))


def test_single_process_instance():
    from deeplearning4j_b200 import DataType
    from deeplearning4j_b200.nd.distributed import ArrayType, DistributedINDArray
    d = DistributedINDArray(ArrayType.CONSTANT, device="cpu").allocateAll(DataType.DOUBLE, 5)
    assert d.numEntries() == 1 and tuple(d.entry(0).t.shape) == (5,)
    d.propagate(torch.ones(2, 2))
    assert torch.equal(d.entry().t, torch.ones(2, 2))
