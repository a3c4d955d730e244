"""RnnOutputLayer takes its rows in (time, example) order when the activations are stored time-major (what the recurrent kernels
produce), so no copy is needed; outputs, score and gradients must equal those of the example-major path."""
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data import DataSet


def _net():
    conf = (nn.NeuralNetConfiguration.Builder().seed(3).updater(nn.Sgd(0.1)).list()
            .layer(nn.RnnOutputLayer("MCXENT", nIn=6, nOut=4, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def test_time_major_rows_give_the_same_output_score_and_gradient():
    g = torch.Generator().manual_seed(0)
    mb, n, T = 5, 6, 7
    base = torch.randn(T, mb, n, generator=g)                     # time-major storage
    x_tm = base.permute(1, 2, 0)                                  # [mb, n, T] view of it
    x_em = x_tm.contiguous()                                      # the same values, example-major storage
    labels = torch.nn.functional.one_hot(torch.randint(0, 4, (mb, T), generator=g), 4).float().permute(0, 2, 1).contiguous()
    mask = (torch.rand(mb, T, generator=g) > 0.3).float()
    a, b = _net(), _net()
    layer = a.layers[0]
    assert layer._is_time_major(x_tm) and not layer._is_time_major(x_em)
    out_tm, out_em = a.output(x_tm), b.output(x_em)
    torch.testing.assert_close(out_tm.t, out_em.t)
    for m in (None, mask):
        ds_tm, ds_em = DataSet(x_tm, labels, None, m), DataSet(x_em, labels, None, m)
        assert abs(a.score(ds_tm) - b.score(ds_em)) < 1e-6
        a.fit(ds_tm); b.fit(ds_em)
        torch.testing.assert_close(a.params().t, b.params().t, rtol=1e-5, atol=1e-6)
