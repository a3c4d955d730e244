"""UI modules (t-SNE, convolutional activations, SameDiff graph) over HTTP, components, binary stats records."""
import json
import urllib.request

import torch

from deeplearning4j_b200.ui import (ChartHistogram, ChartLine, ComponentDiv, ComponentTable, ComponentText, ConvolutionalListenerModule,
                                    SameDiffModule, StaticPageUtil, TsneModule, UIServer, decode_stats, encode_stats)
from deeplearning4j_b200.ui.modules import _grid_image, _png


def _get(url):
    with urllib.request.urlopen(url, timeout=10) as r:
        return r.status, r.headers.get("Content-Type"), r.read()


def test_modules_over_http():
    srv = UIServer(port=0).start()
    try:
        tsne, conv, sdm = TsneModule(), ConvolutionalListenerModule(), SameDiffModule()
        srv.registerModule(tsne).registerModule(conv).registerModule(sdm)
        base = srv.getAddress()
        req = urllib.request.Request(base + "/tsne/upload?sid=s1", data=b"0.5,1.5,cat\n-1,2,dog\n", method="POST")
        assert json.loads(urllib.request.urlopen(req, timeout=10).read())["points"] == 2
        tsne.setCoordinates("s2", torch.tensor([[1.0, 2.0], [3.0, 4.0]]), ["a", "b"])
        assert json.loads(_get(base + "/tsne/sessions")[2]) == ["s1", "s2"]
        assert json.loads(_get(base + "/tsne/coords?sid=s2")[2]) == ["1,2,a", "3,4,b"]
        conv.setImages("c1", 7, [_grid_image(torch.rand(5, 4, 6))])
        st, ct, body = _get(base + "/activations/data?sid=c1&layer=0")
        assert st == 200 and ct == "image/png" and body[:8] == b"\x89PNG\r\n\x1a\n"
        assert json.loads(_get(base + "/activations/info")[2])["c1"] == {"iteration": 7, "layers": 1}
        from deeplearning4j_b200.samediff.core import SameDiff
        sd = SameDiff.create()
        x = sd.var("x", torch.ones(2, 3))
        sd._op("tanh", [x], name="y")
        sdm.setGraph("g", sd)
        g = json.loads(_get(base + "/samediff/graph?name=g")[2])
        assert [o["op"] for o in g["ops"]] == ["tanh"] and g["variables"][0]["shape"] == [2, 3]
    finally:
        srv.stop()


def test_png_encoder_round_trips_through_pillow():
    from PIL import Image
    import io
    img = _grid_image(torch.arange(2 * 3 * 4.0).reshape(2, 3, 4))
    back = Image.open(io.BytesIO(_png(img)))
    assert back.size == (img.shape[1], img.shape[0]) and list(back.getdata())[:img.shape[1]] == img[0].tolist()


def test_components_and_static_page(tmp_path):
    line = ChartLine.Builder("score").addSeries("train", [0, 1, 2], [3.0, 2.0, 1.5]).setYMin(0).build()
    hist = ChartHistogram.Builder("weights").addBin(-1, 0, 3).addBin(0, 1, 5).build()
    table = ComponentTable(["layer", "params"], [["dense", 100], ["out", 20]])
    page = ComponentDiv(None, ComponentText("summary"), line, hist, table)
    d = json.loads(page.toJson())
    assert d["componentType"] == "ComponentDiv" and [c["componentType"] for c in d["components"]] == ["ComponentText", "ChartLine", "ChartHistogram", "ComponentTable"]
    assert d["components"][1]["series"][0]["y"] == [3.0, 2.0, 1.5] and d["components"][3]["content"][1] == ["out", "20"]
    p = tmp_path / "page.html"
    StaticPageUtil.saveHTMLFile(str(p), page)
    html = p.read_text()
    assert html.startswith("<!DOCTYPE html>") and '"ChartHistogram"' in html


def test_binary_stats_record_round_trip():
    rec = {"timestamp": 1700000000123, "iteration": 42, "epoch": 3, "score": 0.125, "learningRates": {"0_W": 1e-3, "0_b": 1e-3},
           "parameters": {"0_W": {"min": -1.0, "max": 2.0, "counts": [1, 5, 9, 2]}}, "memory": {"jvmCurrent": 1, "deviceNames": ["B200"]},
           "performance": {"examplesPerSecond": 1234.5}}
    buf = encode_stats(rec)
    back = decode_stats(buf)
    assert back == rec and len(buf) < len(json.dumps(rec)) + 64
    assert decode_stats(encode_stats({"iteration": 1}))["score"] is None
