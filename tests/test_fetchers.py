"""Dataset iterators: inline Iris, local-file MNIST / CIFAR parsing, synthetic stand-ins, missing-data errors."""
import gzip
import struct

import numpy as np
import pytest
import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data.fetchers import (Cifar10DataSetIterator, EmnistDataSetIterator, IrisDataSetIterator, MnistDataSetIterator,
                                               TinyImageNetDataSetIterator, UciSequenceDataSetIterator)
from deeplearning4j_b200.data.normalizers import NormalizerStandardize


def test_iris_trains_to_high_accuracy():
    it = IrisDataSetIterator(150, 150)
    ds = it.next()
    assert ds.getFeatures().shape == (150, 4) and ds.getLabels().sum(0).tolist() == [50.0, 50.0, 50.0] and it.getLabels()[2] == "Iris-virginica"
    norm = NormalizerStandardize().fit(ds)
    norm.preProcess(ds)
    conf = (nn.NeuralNetConfiguration.Builder().seed(6).updater(nn.Adam(0.05)).weightInit("XAVIER").list()
            .layer(nn.DenseLayer(nIn=4, nOut=8, activation="tanh")).layer(nn.OutputLayer("MCXENT", nIn=8, nOut=3, activation="softmax")).build())
    net = nn.MultiLayerNetwork(conf).init()
    for _ in range(150):
        net.fit(ds)
    from deeplearning4j_b200.data.iterators import ListDataSetIterator
    assert net.evaluate(ListDataSetIterator([ds])).accuracy() > 0.95


def test_mnist_idx_files_and_missing_data(tmp_path):
    d = tmp_path / "MNIST"
    d.mkdir()
    imgs = (np.arange(5 * 28 * 28) % 256).astype(np.uint8).reshape(5, 28, 28)
    labs = np.array([3, 1, 4, 1, 5], dtype=np.uint8)
    with gzip.open(d / "train-images-idx3-ubyte.gz", "wb") as f:
        f.write(struct.pack(">IIII", 0x803, 5, 28, 28) + imgs.tobytes())
    (d / "train-labels-idx1-ubyte").write_bytes(struct.pack(">II", 0x801, 5) + labs.tobytes())
    it = MnistDataSetIterator(2, True, path=str(d), shuffle=False)
    b = list(it)
    assert [x.getFeatures().shape[0] for x in b] == [2, 2, 1] and b[0].getLabels().argmax(1).tolist() == [3, 1]
    assert torch.allclose(b[0].getFeatures()[0], torch.from_numpy(imgs[0].reshape(-1).astype(np.float32) / 255.0))
    with pytest.raises(FileNotFoundError, match="cannot be downloaded"):
        MnistDataSetIterator(2, False, path=str(d))
    with pytest.raises(FileNotFoundError):
        Cifar10DataSetIterator(4, path=str(tmp_path / "nope"))


def test_cifar_binary_and_synthetic_stand_ins(tmp_path):
    d = tmp_path / "CIFAR10"
    d.mkdir()
    rng = np.random.default_rng(0)
    for i in range(1, 6):
        rec = np.concatenate([rng.integers(0, 10, (4, 1), dtype=np.uint8), rng.integers(0, 256, (4, 3072), dtype=np.uint8)], 1)
        rec.tofile(d / f"data_batch_{i}.bin")
    it = Cifar10DataSetIterator(8, True, path=str(d), shuffle=False)
    assert it.numExamples() == 20 and it.next().getFeatures().shape == (8, 3, 32, 32) and it.getLabels()[0] == "airplane"
    syn = MnistDataSetIterator(64, synthetic=True, numExamples=256)
    again = MnistDataSetIterator(64, synthetic=True, numExamples=256)
    assert syn.numExamples() == 256 and torch.equal(syn.x, again.x) and syn.totalOutcomes() == 10 and syn.inputColumns() == 784
    em = EmnistDataSetIterator(EmnistDataSetIterator.Set.LETTERS, 32, synthetic=True, numExamples=128)
    assert em.next().getLabels().shape == (32, 26) and EmnistDataSetIterator.numLabels("balanced") == 47
    tin = TinyImageNetDataSetIterator(16, synthetic=True, numExamples=64)
    assert tin.next().getFeatures().shape == (16, 3, 64, 64) and tin.totalOutcomes() == 200
    uci = UciSequenceDataSetIterator(50, True, synthetic=True)
    ds = uci.next()
    assert ds.getFeatures().shape == (50, 1, 60) and ds.getLabels().shape == (50, 6, 60) and uci.numExamples() == 450
