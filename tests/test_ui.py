"""StatsListener -> StatsStorage (memory, sqlite) -> UIServer JSON endpoints, plus the remote router."""
import json
import urllib.request

import torch

from deeplearning4j_b200 import nn
from deeplearning4j_b200.data.dataset import DataSet
from deeplearning4j_b200.ui import FileStatsStorage, InMemoryStatsStorage, RemoteUIStatsStorageRouter, StatsListener, UIServer


def _net():
    conf = (nn.NeuralNetConfiguration.Builder().seed(1).updater(nn.Adam(1e-2)).list()
            .layer(nn.DenseLayer(nIn=4, nOut=8, activation="relu")).layer(nn.OutputLayer("MCXENT", nIn=8, nOut=3, activation="softmax")).build())
    return nn.MultiLayerNetwork(conf).init()


def _data():
    g = torch.Generator().manual_seed(0)
    return DataSet(torch.randn(16, 4, generator=g), torch.nn.functional.one_hot(torch.randint(0, 3, (16,), generator=g), 3).float())


def _get(url):
    return json.loads(urllib.request.urlopen(url, timeout=5).read())


def test_stats_listener_storage_and_server(tmp_path):
    mem, fil = InMemoryStatsStorage(), FileStatsStorage(str(tmp_path / "stats.db"))
    events = []
    mem.registerStatsStorageListener(lambda ev: events.append(ev.eventType))
    net = _net()
    sl = StatsListener(mem, 2)
    net.setListeners(sl, StatsListener(fil, 1, sessionID="file-session"))
    ds = _data()
    for _ in range(6):
        net.fit(ds)
    sid = sl.getSessionID()
    assert mem.listSessionIDs() == [sid] and mem.getNumUpdateRecordsFor(sid) == 3 and events.count("PostUpdate") == 3 and events[0] == "PostStaticInfo"
    static = mem.getStaticInfo(sid, StatsListener.TYPE_ID, sl.getWorkerID())
    assert static["numParams"] == net.numParams() and [l["type"] for l in static["layers"]] == ["DenseLayer", "OutputLayer"]
    last = mem.getLatestUpdate(sid, StatsListener.TYPE_ID)
    assert set(last["parameters"]) == {"0_W", "0_b", "1_W", "1_b"} and sum(last["parameters"]["0_W"]["histogram"]["counts"]) == 32
    assert last["updateRatios"]["0_W"] > 0 and last["learningRates"]["1_b"] == 1e-2 and last["performance"]["examplesPerSecond"] > 0
    fil.close()
    reopened = FileStatsStorage(str(tmp_path / "stats.db"))
    assert reopened.getNumUpdateRecordsFor("file-session") == 6
    srv = UIServer(port=0).start()
    try:
        srv.attach(mem)
        srv.attach(reopened)
        base = srv.getAddress()
        assert set(_get(base + "/train/sessions")) == {sid, "file-session"}
        ov = _get(base + f"/train/overview?sid={sid}")
        assert [p[0] for p in ov["scores"]] == [0, 2, 4] and ov["lastIteration"] == 4
        model = _get(base + "/train/model?sid=file-session")
        assert model["numParams"] == net.numParams() and "1_W" in model["gradients"]
        assert "hardware" in _get(base + f"/train/system?sid={sid}")
        assert b"Training overview" in urllib.request.urlopen(base + "/", timeout=5).read()
        # remote routing into the server
        srv.enableRemoteListener()
        net2 = _net()
        net2.setListeners(StatsListener(RemoteUIStatsStorageRouter(base), 1, sessionID="remote"))
        for _ in range(2):
            net2.fit(ds)
        assert "remote" in _get(base + "/train/sessions") and len(_get(base + "/train/overview?sid=remote")["scores"]) == 2
    finally:
        srv.stop()
