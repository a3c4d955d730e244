"""ParallelInference: batched / sequential / in-place modes give the model's own outputs."""
import threading

import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.parallel.inference import InferenceMode, InplaceParallelInference, LoadBalanceMode, ParallelInference


def _net():
    conf = (nn.NeuralNetConfiguration.Builder().seed(3).list()
            .layer(nn.DenseLayer(nIn=6, nOut=12, activation="tanh"))
            .layer(nn.OutputLayer("MCXENT", nIn=12, nOut=4, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def test_batched_mode_coalesces_and_matches_direct_output():
    net = _net()
    pi = (ParallelInference.Builder(net).workers(2).inferenceMode(InferenceMode.BATCHED).batchLimit(16).queueLimit(128)
          .loadBalanceMode(LoadBalanceMode.FIFO).build())
    g = torch.Generator().manual_seed(0)
    xs = [torch.randn(1 + i % 3, 6, generator=g) for i in range(40)]
    results = [None] * len(xs)

    def call(i):
        results[i] = pi.output(xs[i]).t
    ts = [threading.Thread(target=call, args=(i,)) for i in range(len(xs))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for x, r in zip(xs, results):
        assert torch.allclose(r, net.output(x).t, atol=1e-6)
    st = pi.stats()
    assert sum(s["examples"] for s in st) == sum(x.shape[0] for x in xs) and sum(s["batches"] for s in st) <= len(xs)
    pi.shutdown()


def test_sequential_round_robin_inplace_and_update_model():
    net = _net()
    pi = ParallelInference(net, workers=2, inferenceMode=InferenceMode.SEQUENTIAL, loadBalanceMode=LoadBalanceMode.ROUND_ROBIN)
    x = torch.randn(5, 6, generator=torch.Generator().manual_seed(1))
    outs = pi.outputBatches([x, x, x, x])
    assert all(torch.allclose(o.t, net.output(x).t, atol=1e-6) for o in outs)
    assert [s["batches"] for s in pi.stats()] == [2, 2]
    other = _net()
    other.setParams(net.params().t * 0.5 if hasattr(net.params(), "t") else net.params() * 0.5)
    pi.updateModel(other)
    assert torch.allclose(pi.output(x).t, other.output(x).t, atol=1e-6)
    pi.shutdown()
    ip = InplaceParallelInference(net, workers=3)
    assert torch.allclose(ip.output(x).t, net.output(x).t, atol=1e-6) and len(ip.getCurrentModelsFromWorkers()) == 3
