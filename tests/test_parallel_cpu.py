"""Host-side data-parallel logic on CPU ranks (gloo, world_size 2): config-1 MLP with threshold-encoded
sharing, gradient averaging, classic parameter averaging, and the codec round trip."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _mlp(seed=123, updater=None):
    from deeplearning4j_b200 import nn
    conf = (nn.NeuralNetConfiguration.Builder().seed(seed).updater(updater or nn.Adam(1e-3)).weightInit("XAVIER").list()
            .layer(nn.DenseLayer(nIn=784, nOut=512, activation="relu"))
            .layer(nn.DenseLayer(nIn=512, nOut=512, activation="relu"))
            .layer(nn.OutputLayer("MCXENT", nIn=512, nOut=10, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def _data(seed, n=128):
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(n, 784, generator=g)
    y = torch.nn.functional.one_hot(torch.randint(0, 10, (n,), generator=g), 10).float()
    return x, y


def _worker_threshold(rank, world, out_dir):
    import torch.distributed as dist
    from deeplearning4j_b200.parallel.wrapper import ParallelWrapper, TrainingMode
    from deeplearning4j_b200.parallel.sharing import FixedThresholdAlgorithm
    net = _mlp(seed=123 + rank)          # different init per rank: wrapper must broadcast rank 0's parameters
    pw = (ParallelWrapper.Builder(net).workers(world).trainingMode(TrainingMode.SHARED_GRADIENTS)
          .thresholdAlgorithm(FixedThresholdAlgorithm(1e-3)).build())
    x, y = _data(7 + rank)
    s0 = None
    for i in range(25):
        net.fit(x, y)
        if i == 0:
            s0 = net.score()
    p = net.flat_params.clone()
    gathered = [torch.zeros_like(p) for _ in range(world)]
    dist.all_gather(gathered, p)
    assert all(torch.equal(gathered[0], g) for g in gathered), "replicas diverged"
    assert net.score() < s0
    assert pw.sharing.bytes_sent > 0
    if rank == 0:
        from deeplearning4j_b200.nn import ModelSerializer
        path = os.path.join(out_dir, "model.zip")
        ModelSerializer.writeModel(net, path, True)
        net2 = ModelSerializer.restoreMultiLayerNetwork(path)
        assert torch.equal(net2.flat_params, net.flat_params)
        assert torch.equal(net2.updater.state, net.updater.state)
        assert net2.conf.toJson() == net.conf.toJson()
        torch.save({"s0": s0, "s1": net.score()}, os.path.join(out_dir, "ok.pt"))


def _worker_averaging(rank, world, out_dir, freq):
    import torch.distributed as dist
    from deeplearning4j_b200 import nn
    from deeplearning4j_b200.parallel.wrapper import ParallelWrapper
    net = _mlp(seed=5 + rank, updater=nn.Sgd(0.1))
    ParallelWrapper.Builder(net).workers(world).averagingFrequency(freq).build()
    x, y = _data(11 + rank)
    for i in range(2 * max(freq, 1)):
        net.fit(x, y)
    p = net.flat_params.clone()
    gathered = [torch.zeros_like(p) for _ in range(world)]
    dist.all_gather(gathered, p)
    assert all(torch.allclose(gathered[0], g, atol=1e-7) for g in gathered)
    if freq == 1 and rank == 0:
        # gradient averaging with SGD == single process on the concatenated batch
        ref = _mlp(seed=5, updater=nn.Sgd(0.1))
        xs = torch.cat([_data(11 + r)[0] for r in range(world)])
        ys = torch.cat([_data(11 + r)[1] for r in range(world)])
        for i in range(2):
            ref.fit(xs, ys)
        assert torch.allclose(ref.flat_params, net.flat_params, atol=2e-5), float((ref.flat_params - net.flat_params).abs().max())
    if rank == 0:
        torch.save({"ok": True}, os.path.join(out_dir, f"avg{freq}.pt"))


def test_threshold_sharing_world2(tmp_path):
    from deeplearning4j_b200.parallel.wrapper import launch
    launch(_worker_threshold, 2, str(tmp_path), backend="gloo", port=29611)
    r = torch.load(tmp_path / "ok.pt")
    assert r["s1"] < r["s0"]


@pytest.mark.parametrize("freq", [1, 3])
def test_averaging_world2(tmp_path, freq):
    from deeplearning4j_b200.parallel.wrapper import launch
    launch(_worker_averaging, 2, str(tmp_path), freq, backend="gloo", port=29620 + freq)
    assert (tmp_path / f"avg{freq}.pt").exists()


@pytest.mark.parametrize("n", [1, 15, 16, 17, 1000, 4099])
def test_codec_roundtrip(n):
    from deeplearning4j_b200.parallel import codec
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g) * 2e-3
    tau = 1e-3
    for enc, dec in ((codec.threshold_encode, codec.threshold_decode), (codec.bitmap_encode, codec.bitmap_decode)):
        r = x.clone()
        msg = enc(r, tau)
        assert int(msg[1]) == n and msg.dtype == torch.int32
        out = torch.zeros(n)
        dec(msg, out)
        assert torch.allclose(out + r, x, atol=1e-7)
        big = x.abs() >= tau
        assert torch.allclose(out[big], torch.sign(x[big]) * tau)
    # sparse payload is in ascending index order and capacity-limited
    r = x.clone()
    msg = codec.threshold_encode(r, tau, capacity=3)
    k = int(msg[0])
    assert k <= 3 and msg.numel() == 4 + k
    idx = msg[4:].abs()
    assert torch.equal(idx, torch.sort(idx).values)


def test_threshold_algorithms():
    from deeplearning4j_b200.parallel.sharing import AdaptiveThresholdAlgorithm, ResidualClippingPostProcessor, TargetSparsityThresholdAlgorithm
    a = AdaptiveThresholdAlgorithm(1e-3, 1e-4, 1e-2, 0.9)
    t0 = a.calculateThreshold(0, 0, None, False, None, None)
    assert t0 == 1e-3
    assert a.calculateThreshold(1, 0, t0, False, 0.5, None) > t0        # too dense -> raise the threshold
    assert a.calculateThreshold(1, 0, t0, False, 1e-6, None) < t0       # too sparse -> lower it
    t = TargetSparsityThresholdAlgorithm(1e-4, 1e-3, 0.9)
    assert t.calculateThreshold(1, 0, 1e-4, False, 1e-2, None) > 1e-4
    r = torch.tensor([10.0, -10.0, 0.001])
    ResidualClippingPostProcessor(5, 5).processResidual(5, 0, 1e-3, r)
    assert float(r.abs().max()) <= 5e-3 + 1e-9
