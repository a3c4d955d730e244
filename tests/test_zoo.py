"""Every zoo model builds, runs a forward pass and (for a few) trains / round-trips through JSON."""
import pytest
import torch

from deeplearning4j_b200.data.dataset import DataSet
from deeplearning4j_b200.models import zoo_cnn as Z
from deeplearning4j_b200.models.zoo import ResNet50, TextGenerationLSTM

CASES = {"LeNet": (dict(inputShape=(1, 28, 28), numClasses=10), 1256080), "SimpleCNN": (dict(inputShape=(3, 48, 48), numClasses=7), None),
         "AlexNet": (dict(inputShape=(3, 224, 224), numClasses=10), None), "VGG16": (dict(inputShape=(3, 32, 32), numClasses=10), None),
         "VGG19": (dict(inputShape=(3, 32, 32), numClasses=10), None), "Darknet19": (dict(inputShape=(3, 64, 64), numClasses=10), None),
         "TinyYOLO": (dict(inputShape=(3, 64, 64), numClasses=3), None), "YOLO2": (dict(inputShape=(3, 64, 64), numClasses=3), None),
         "SqueezeNet": (dict(inputShape=(3, 96, 96), numClasses=10), None), "UNet": (dict(inputShape=(3, 32, 32)), None),
         "Xception": (dict(inputShape=(3, 96, 96), numClasses=10), None), "InceptionResNetV1": (dict(inputShape=(3, 160, 160), numClasses=10), None),
         "FaceNetNN4Small2": (dict(inputShape=(3, 96, 96), numClasses=10), None),
         "NASNet": (dict(inputShape=(3, 32, 32), numClasses=10, numBlocks=2, penultimateFilters=240, stemFilters=32), None)}


@pytest.mark.parametrize("name", sorted(CASES))
def test_zoo_model_builds_and_runs(name):
    kw, n_params = CASES[name]
    net = Z.ALL_MODELS[name](**kw).init()
    c, h, w = kw["inputShape"]
    x = torch.randn(2, c, h, w, generator=torch.Generator().manual_seed(0))
    if name in ("LeNet", "VGG16", "VGG19"):
        x = x.reshape(2, -1)                                   # convolutionalFlat input type
    out = net.output(x)
    out = (out[0] if isinstance(out, (list, tuple)) else out).t
    assert out.shape[0] == 2 and bool(torch.isfinite(out).all())
    if n_params is not None:
        assert net.numParams() == n_params
    if name in ("LeNet", "SimpleCNN", "SqueezeNet", "Darknet19", "NASNet", "FaceNetNN4Small2"):
        assert abs(float(out.sum(1).mean()) - 1.0) < 1e-3      # class probabilities


def test_vgg16_parameter_count_at_imagenet_size():
    conf = Z.VGG16(numClasses=1000).conf()
    from deeplearning4j_b200.nn.conf.graphconf import LayerVertex
    n = sum(sum(s.numel for s in v.layer.param_specs()) for v in conf.vertices.values() if isinstance(v, LayerVertex))
    assert n == 138357544                                       # the canonical VGG-16 size


def test_lenet_trains_and_yolo_json_round_trip():
    net = Z.LeNet(numClasses=4, inputShape=(1, 12, 12)).init()
    g = torch.Generator().manual_seed(1)
    y = torch.randint(0, 4, (32,), generator=g)
    x = torch.randn(32, 1, 12, 12, generator=g) + y.reshape(-1, 1, 1, 1).float()
    ds = DataSet(x.reshape(32, -1), torch.nn.functional.one_hot(y, 4).float())
    s0 = net.score(ds)
    for _ in range(15):
        net.fit(ds)
    assert net.score(ds) < s0
    conf = Z.TinyYOLO(numClasses=2, inputShape=(3, 64, 64)).conf()
    from deeplearning4j_b200.nn.conf.graphconf import ComputationGraphConfiguration
    back = ComputationGraphConfiguration.fromJson(conf.toJson())
    assert back.toJson() == conf.toJson() and "outputs" in back.vertices


def test_zoo_builder_api():
    m = ResNet50.builder().numClasses(10).seed(7).build()
    assert m.numClasses == 10 and m.seed == 7 and m.modelType() == "ResNet50" and m.metaData()["zooType"] == "CNN"
    with pytest.raises(IOError):
        m.initPretrained()
    assert TextGenerationLSTM(totalUniqueCharacters=30).metaData()["zooType"] == "RNN"
    with pytest.raises(ValueError):
        Z.NASNet(penultimateFilters=100)
