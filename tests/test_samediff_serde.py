"""FlatBuffers (.fb), SDNB and SDZ round trips of a SameDiff training graph (tiny BERT), CPU only."""
import os
import struct

import numpy as np
import pytest
import torch

from deeplearning4j_b200 import DataType
from deeplearning4j_b200.models.bert import BertConfig, build_bert_mlm
from deeplearning4j_b200.nn.updaters import Adam
from deeplearning4j_b200.samediff.core import SameDiff
from deeplearning4j_b200.samediff.serde import flatbuffers as fb
from deeplearning4j_b200.samediff.serde import sdnb


@pytest.fixture(scope="module")
def trained():
    cfg = BertConfig(vocabSize=512, hidden=64, layers=2, heads=4, ffn=128, maxPositions=32)
    B, T = 2, 32
    sd = build_bert_mlm(cfg, B, T, Adam(1e-3), DataType.FLOAT)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocabSize, (B, T), generator=g)
    pos = torch.randperm(B * T, generator=g)[:10].sort().values
    ph = {"tokens": tok, "maskedPositions": pos, "maskedLabels": tok.reshape(-1)[pos]}
    for _ in range(3):
        sd.fit(ph, 1)
    return sd, ph


def _same_graph(a, b):
    assert list(a.variables) == list(b.variables)
    assert [(o.name, o.opName, o.inputs, o.outputs, o.args) for o in a.ops] == \
           [(o.name, o.opName, o.inputs, o.outputs, o.args) for o in b.ops]
    for n, arr in a.arrays.items():
        if n in b.arrays:
            assert torch.equal(arr.cpu(), b.arrays[n].cpu()), n
    assert a.lossVariables == b.lossVariables


def test_flatbuffers_wire_format():
    obj = {"id": 7, "name": "n", "opType": 21, "opNum": -5, "input": [1, 2, 3], "extraParams": [0.5, 1.5],
           "inputPaired": [{"first": 1, "second": 0}, {"first": 0, "second": 2}], "outputNames": ["a", "bc"],
           "extraBools": [True, False], "scalar": {"shape": [2], "buffer": b"\x01\x02\x03\x04\x05\x06\x07\x08", "dtype": 5}}
    raw = fb.encode("FlatNode", obj)
    root = struct.unpack_from("<I", raw, 0)[0]
    vt = root - struct.unpack_from("<i", raw, root)[0]
    assert struct.unpack_from("<H", raw, vt)[0] % 2 == 0 and root % 8 == 0          # table holds a long -> 8-aligned
    back = fb.decode("FlatNode", raw, raw_bytes=False)
    assert back["id"] == 7 and back["opNum"] == -5 and back["input"] == [1, 2, 3] and back["extraParams"] == [0.5, 1.5]
    assert back["inputPaired"][1] == {"first": 0, "second": 2} and back["outputNames"] == ["a", "bc"]
    assert back["extraBools"] == [True, False] and back["device"] == 0 and back["opName"] is None
    assert bytes(bytearray(x & 0xFF for x in back["scalar"]["buffer"])) == b"\x01\x02\x03\x04\x05\x06\x07\x08"


def test_fb_round_trip_continues_training_identically(trained):
    sd, ph = trained
    buf = sd.asFlatBuffers(True)
    sd2 = SameDiff.fromFlatBuffers(buf)
    _same_graph(sd, sd2)
    assert torch.equal(sd._training.updater.state, sd2._training.updater.state)
    assert sd2.trainingConfig.iterationCount == sd.trainingConfig.iterationCount
    assert sd2.asFlatBuffers(True) == buf                                            # byte-stable
    out1 = sd.output(ph, sd.lossVariables[0])[sd.lossVariables[0]]
    out2 = sd2.output(ph, sd.lossVariables[0])[sd.lossVariables[0]]
    assert torch.equal(out1.t, out2.t)


def test_sdnb_header_manifest_and_round_trip(trained, tmp_path):
    sd, ph = trained
    p = str(tmp_path / "model.sdnb")
    sdnb.save(sd, p, True, appendThreshold=50_000)
    raw = open(p, "rb").read()
    assert raw[:4] == b"SDNB"
    ver, moff, mlen, goff = struct.unpack(">iqqq", raw[4:32])
    assert (ver, goff) == (1, 32) and moff + mlen == len(raw)
    assert raw[moff:moff + 2] == b"\xac\xed"                                          # Java object stream
    manifest = sdnb.read_manifest(raw[moff:moff + mlen])
    assert manifest and all(32 < off < moff and ln > 0 for off, ln in manifest.values())
    name, (off, ln) = next(iter(manifest.items()))
    assert np.array_equal(np.frombuffer(raw[off:off + ln], "<f4"), sd.arrays[name].reshape(-1).numpy())
    sd2 = SameDiff.load(p, True)
    _same_graph(sd, sd2)
    assert torch.equal(sd._training.updater.state, sd2._training.updater.state)


def test_sharded_sdnb_and_sdz(trained, tmp_path):
    sd, ph = trained
    files = sdnb.save(sd, str(tmp_path / "big.sdnb"), True, maxShardBytes=150_000, appendThreshold=20_000)
    assert len(files) > 2 and files[0].endswith(f".shard0-of-{len(files)}.sdnb")
    _same_graph(sd, SameDiff.load(str(tmp_path / "big.sdnb")))
    os.remove(files[-1])
    with pytest.raises(FileNotFoundError):
        SameDiff.load(str(tmp_path / "big.sdnb"))
    z = str(tmp_path / "m.sdz")
    sd.saveAsSDZ(z)
    sd3 = SameDiff.loadSDZ(z)
    _same_graph(sd, sd3)
    l_a = sd.fit(ph, 1).losses[-1][-1]
    l_b = sd3.fit(ph, 1).losses[-1][-1]
    assert l_a == l_b


def test_java_manifest_codec():
    m = {"w": (32, 1 << 33), "layer/b": (40, 0)}
    raw = sdnb.write_manifest(m)
    assert raw[:4] == b"\xac\xed\x00\x05" and b"java.util.LinkedHashMap" in raw and b"org.nd4j.common.primitives.Pair" in raw
    assert sdnb.read_manifest(raw) == m
    assert sdnb.read_manifest(sdnb.write_manifest({})) == {}
