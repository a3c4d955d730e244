"""Failure detection and checkpoint recovery on CPU ranks (gloo): the failure is made on the host (a rank raises / exits), the
survivor learns of it through the heartbeat store before its next step, and a relaunched job resumes from the last checkpoint."""
import os
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _net(seed=5):
    from deeplearning4j_b200 import nn
    conf = (nn.NeuralNetConfiguration.Builder().seed(seed).updater(nn.Adam(1e-2)).list()
            .layer(nn.DenseLayer(nIn=8, nOut=16, activation="relu"))
            .layer(nn.OutputLayer("MCXENT", nIn=16, nOut=3, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def _batches(n, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        x = torch.rand(16, 8, generator=g)
        y = torch.nn.functional.one_hot(torch.randint(0, 3, (16,), generator=g), 3).float()
        out.append((x, y))
    return out


def _worker(rank, world, port, out_dir, fail_at):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deeplearning4j_b200.parallel.elastic import ElasticTrainer, PeerFailure
    from deeplearning4j_b200.parallel.wrapper import ParallelWrapper, TrainingMode
    net = _net()
    ParallelWrapper.Builder(net).workers(world).trainingMode(TrainingMode.AVERAGING).averagingFrequency(1).build()
    trainer = ElasticTrainer(net, os.path.join(out_dir, "ckpt"), checkpointEvery=4, heartbeatTimeout=30.0)     # the failure is announced, not timed out
    batches = _batches(40, 11 + rank)
    result = {"rank": rank}

    def stepper():
        for i, b in enumerate(batches):
            if rank == 1 and i == fail_at:
                raise RuntimeError("injected host failure")           # the failing rank leaves between steps
            yield b
    try:
        trainer.fit(stepper())
        result["outcome"] = "finished"
    except PeerFailure as e:
        result["outcome"] = "peer_failure"
        result["failed_rank"] = e.rank
        result["reason"] = e.reason
    except RuntimeError as e:
        result["outcome"] = "self_failure"
        result["reason"] = str(e)
    result["iterations"] = net.getIterationCount()
    torch.save(result, os.path.join(out_dir, f"result{rank}.pt"))
    # no collective may follow a failure: leave without the usual barrier
    os._exit(0)


def test_rank_failure_is_detected_and_training_resumes_from_checkpoint(tmp_path):
    out = str(tmp_path)
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, 29611, out, 10)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive(), "worker did not finish"
    r0, r1 = torch.load(os.path.join(out, "result0.pt")), torch.load(os.path.join(out, "result1.pt"))
    assert r1["outcome"] == "self_failure" and "injected" in r1["reason"]
    assert r0["outcome"] == "peer_failure" and r0["failed_rank"] == 1 and "injected" in r0["reason"]
    assert r0["iterations"] == 10                         # the survivor stopped before launching step 10
    # relaunch with the surviving world (one rank): resume from the newest checkpoint and continue
    from deeplearning4j_b200.parallel.elastic import ElasticTrainer
    net = _net(seed=99)                                    # different init: everything must come from the checkpoint
    trainer = ElasticTrainer(net, os.path.join(out, "ckpt"), checkpointEvery=4)
    it = trainer.resume()
    assert it == 8 and net.getIterationCount() == 9       # newest checkpoint: written when iteration index 8 finished (9 done)
    ref = _net()
    done = trainer.fit(_batches(5, 3))
    assert done == 5 and net.getIterationCount() == 14
    assert ElasticTrainer.lastCheckpointIteration(os.path.join(out, "ckpt")) == 12
    assert not torch.equal(net.flat_params, ref.flat_params)


def test_heartbeat_timeout_and_watchdog_without_a_device():
    from deeplearning4j_b200.parallel.elastic import CudaWatchdog, HeartbeatMonitor, PeerFailure, StepTimeout

    class Store(dict):
        def set(self, k, v): self[k] = v.encode() if isinstance(v, str) else v
        def get(self, k): return self[k]
    s = Store()
    a, b = HeartbeatMonitor(s, rank=0, world=2, timeout=0.2), HeartbeatMonitor(s, rank=1, world=2, timeout=0.2)
    a.beat(0)
    b.beat(0)
    a.check()
    time.sleep(0.3)
    a.beat(1)
    with pytest.raises(PeerFailure, match="no heartbeat"):
        a.check()                                          # rank 1 stopped publishing
    b.announce_failure("OOM in data loader")
    with pytest.raises(PeerFailure, match="OOM"):
        a.check()

    class NeverDone:
        def query(self): return False
    wd = CudaWatchdog(deadline=0.1, poll=0.02)
    wd.arm(NeverDone())
    time.sleep(0.3)
    with pytest.raises(StepTimeout):
        wd.check()
    wd.close()


def test_device_status_is_surfaced_through_elastic_trainer(tmp_path):
    """A bounded device-side wait that gave up is reported one step later: the poller clears the sticky status word, zeroes the
    gradients the kernel left behind and the trainer raises.  The device access is replaced by a host stand-in (no GPU)."""
    from deeplearning4j_b200.parallel.elastic import ElasticTrainer, PeerFailure
    from deeplearning4j_b200.parallel.fused import DeviceStatusPoller

    class FakeEvent:
        def query(self): return True
        def synchronize(self): pass

    class FakePoller(DeviceStatusPoller):
        word = 0
        cleared = 0

        def _queue_copy(self):
            return FakeEvent(), torch.tensor([self.word], dtype=torch.int32)

        def _clear_word(self):
            self.cleared += 1
            self.word = 0

    net = _net()
    poller = FakePoller(net.flat_grads)

    class Hook:                        # stands in for FusedAveraging: steps nothing, reports through the poller
        class fused:
            status = poller

        def __call__(self, model):
            poller.check()
            poller.snapshot()
            if model.iterationCount == 2:
                poller.word = 4        # the *next* snapshot sees an expired peer wait
            return False
    net.gradient_hook = Hook()
    trainer = ElasticTrainer(net, str(tmp_path / "ckpt"), checkpointEvery=100)
    net.flat_grads.fill_(3.0)
    with pytest.raises(PeerFailure):
        trainer.fit(_batches(8, 1))
    assert poller.cleared == 1 and poller.word == 0
    assert float(net.flat_grads.abs().sum()) == 0.0          # stale gradients were dropped
    assert net.getIterationCount() < 8
    # the word is clear again: training continues
    done = trainer.fit(_batches(2, 2))
    assert done == 2
