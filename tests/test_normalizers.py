"""Normalizers: statistics, transform/revert, NormalizerSerializer stream layout, ModelSerializer integration."""
import io
import struct

import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data.dataset import DataSet, MultiDataSet
from deeplearning4j_b200.data.iterators import ListDataSetIterator
from deeplearning4j_b200.data.normalizers import (ImagePreProcessingScaler, MultiNormalizerStandardize, NormalizerMinMaxScaler,
                                                  NormalizerSerializer, NormalizerStandardize, VGG16ImagePreProcessor)


def _sets(seed=0):
    g = torch.Generator().manual_seed(seed)
    return [DataSet(torch.randn(20, 5, generator=g) * 3 + 2, torch.randn(20, 2, generator=g) * 10) for _ in range(4)]


def test_standardize_fit_transform_revert_and_stream():
    sets = _sets()
    allx = torch.cat([d.getFeatures().t if hasattr(d.getFeatures(), "t") and not isinstance(d.getFeatures(), torch.Tensor) else d.getFeatures() for d in sets])
    n = NormalizerStandardize().fitLabel(True)
    n.fit(ListDataSetIterator(sets))
    assert torch.allclose(n.mean_, allx.mean(0), atol=1e-5) and torch.allclose(n.std_, allx.std(0, unbiased=False), atol=1e-5)
    ds = DataSet(allx.clone(), torch.zeros(80, 2))
    n.preProcess(ds)
    f = ds.getFeatures()
    f = f if isinstance(f, torch.Tensor) else f.t
    assert torch.allclose(f.mean(0), torch.zeros(5), atol=1e-5) and torch.allclose(f.std(0, unbiased=False), torch.ones(5), atol=1e-4)
    n.revert(ds)
    f = ds.getFeatures()
    f = f if isinstance(f, torch.Tensor) else f.t
    assert torch.allclose(f, allx, atol=1e-4)
    bio = io.BytesIO()
    NormalizerSerializer.write(n, bio)
    raw = bio.getvalue()
    assert raw[:2] == struct.pack(">H", 10) and raw[2:12] == b"NORMALIZER" and raw[12:16] == struct.pack(">i", 1)
    assert raw[16:18] == struct.pack(">H", 11) and raw[18:29] == b"STANDARDIZE" and raw[29] == 1
    n2 = NormalizerSerializer.restore(io.BytesIO(raw))
    assert torch.equal(n2.mean_, n.mean_) and torch.equal(n2.labelStd, n.labelStd) and n2.isFitLabel()


def test_min_max_image_vgg_and_multi(tmp_path):
    sets = _sets(1)
    mm = NormalizerMinMaxScaler(-1, 1)
    mm.fit(ListDataSetIterator(sets))
    x = sets[0].getFeatures()
    z = mm.transform(x)
    zt = z if isinstance(z, torch.Tensor) else z.t
    assert float(zt.min()) >= -1 - 1e-6 and float(zt.max()) <= 1 + 1e-6
    back = mm.revertFeatures(z)
    assert torch.allclose(back if isinstance(back, torch.Tensor) else back.t, x if isinstance(x, torch.Tensor) else x.t, atol=1e-4)
    p = str(tmp_path / "mm.bin")
    NormalizerSerializer.write(mm, p)
    mm2 = NormalizerSerializer.restore(p)
    assert mm2.targetMin == -1 and torch.equal(mm2.max_, mm.max_)
    img = ImagePreProcessingScaler(0, 1)
    assert float(img.transform(torch.full((1, 3, 2, 2), 255.0)).max()) == 1.0
    bio = io.BytesIO()
    NormalizerSerializer.write(img, bio)
    assert NormalizerSerializer.restore(bio.getvalue()).maxPixelVal == 255.0
    v = VGG16ImagePreProcessor().transform(torch.zeros(1, 3, 2, 2))
    assert abs(float(v[0, 0, 0, 0]) + 123.68) < 1e-4
    g = torch.Generator().manual_seed(2)
    mds = [MultiDataSet([torch.randn(10, 3, generator=g) + 5, torch.randn(10, 4, generator=g) * 2], [torch.randn(10, 1, generator=g)]) for _ in range(3)]
    mn = MultiNormalizerStandardize()
    mn.fit(mds)
    out = mn.preProcess(mds[0])
    f0 = out.getFeatures()[0]
    f0 = f0 if isinstance(f0, torch.Tensor) else f0.t
    assert abs(float(f0.mean())) < 0.6 and mn.numInputs() == 2
    bio = io.BytesIO()
    NormalizerSerializer.write(mn, bio)
    mn2 = NormalizerSerializer.restore(bio.getvalue())
    assert torch.equal(mn2.inputs[1].std_, mn.inputs[1].std_)


def test_time_series_mask_statistics_and_model_zip(tmp_path):
    x = torch.zeros(2, 3, 4)
    x[0, :, :2] = torch.tensor([[1.0, 3.0], [2.0, 4.0], [0.0, 0.0]])
    x[1] = 100.0
    mask = torch.tensor([[1.0, 1, 0, 0], [0, 0, 0, 0]])
    n = NormalizerStandardize()
    n.fit(DataSet(x, None, mask, None))
    assert torch.allclose(n.mean_, torch.tensor([2.0, 3.0, 0.0])) and torch.allclose(n.std_, torch.tensor([1.0, 1.0, 0.0]))
    conf = (nn.NeuralNetConfiguration.Builder().list().layer(nn.OutputLayer("MSE", nIn=3, nOut=1, activation="identity")).build())
    net = nn.MultiLayerNetwork(conf).init()
    p = str(tmp_path / "m.zip")
    nn.ModelSerializer.writeModel(net, p, True, n)
    n2 = nn.ModelSerializer.restoreNormalizerFromFile(p)
    assert torch.equal(n2.mean_, n.mean_)
