"""The plain-Python HDF5 subset (``importers/hdf5.py``) and Keras ``.h5`` import through it (reference:
``deeplearning4j-modelimport/.../keras/Hdf5Archive.java``, ``KerasModelImport.importKerasModelAndWeights(String)``).  No HDF5
library exists here, so the files are written by the module's own writer, structure by structure as the format specification lays
them out; the byte-level test pins the parts of the layout that other readers rely on."""
import json
import struct

import numpy as np
import pytest
import torch

from deeplearning4j_b200.importers.hdf5 import Hdf5Archive, Hdf5File, Hdf5FormatError, Hdf5Writer


def _keras_file(tmp_path, full=True):
    g = np.random.default_rng(0)
    k1, b1 = g.standard_normal((6, 5)).astype(np.float32), g.standard_normal(5).astype(np.float32)
    k2, b2 = g.standard_normal((5, 3)).astype(np.float32), g.standard_normal(3).astype(np.float32)
    cfg = {"class_name": "Sequential", "config": {"name": "seq", "layers": [
        {"class_name": "Dense", "config": {"name": "dense", "units": 5, "activation": "tanh", "use_bias": True, "batch_input_shape": [None, 6]}},
        {"class_name": "Dense", "config": {"name": "dense_1", "units": 3, "activation": "softmax", "use_bias": True}}]}}
    w = Hdf5Writer()
    root = "model_weights" if full else ""
    if full:
        w.attr("", "model_config", json.dumps(cfg))
        w.attr("", "keras_version", "2.9.0")
        w.attr("", "backend", "tensorflow")
        w.attr("", "training_config", json.dumps({"loss": "categorical_crossentropy", "optimizer_config": {"class_name": "Adam", "config": {}}}))
    w.group(root)
    w.attr(root, "layer_names", [b"dense", b"dense_1"])
    for lname, (k, b) in (("dense", (k1, b1)), ("dense_1", (k2, b2))):
        w.attr(f"{root}/{lname}", "weight_names", [f"{lname}/kernel:0".encode(), f"{lname}/bias:0".encode()])
        w.dataset(f"{root}/{lname}/{lname}/kernel:0", k)
        w.dataset(f"{root}/{lname}/{lname}/bias:0", b)
    p = tmp_path / ("model.h5" if full else "weights.h5")
    w.save(str(p))
    return str(p), cfg, (k1, b1, k2, b2)


def test_layout_of_the_written_file(tmp_path):
    p, _, _ = _keras_file(tmp_path)
    raw = open(p, "rb").read()
    assert raw[:8] == b"\x89HDF\r\n\x1a\n" and raw[8] == 0 and raw[13] == 8 and raw[14] == 8       # superblock v0, 8-byte offsets / lengths
    eof = struct.unpack_from("<Q", raw, 40)[0]
    assert eof == len(raw)
    root_hdr = struct.unpack_from("<Q", raw, 64)[0]
    assert raw[root_hdr] == 1                                                                    # version-1 object header
    btree, heap = struct.unpack_from("<QQ", raw, 80)                                             # cached in the root symbol-table entry
    assert raw[btree:btree + 4] == b"TREE" and raw[heap:heap + 4] == b"HEAP"
    assert raw.count(b"SNOD") >= 4 and b"GCOL" in raw


def test_groups_datasets_and_attributes(tmp_path):
    p, cfg, (k1, b1, k2, b2) = _keras_file(tmp_path)
    with Hdf5File(p) as f:
        assert f.keys() == ["model_weights"]
        mw = f["model_weights"]
        assert mw.keys() == ["dense", "dense_1"]
        assert [s.decode() for s in mw.attrs["layer_names"]] == ["dense", "dense_1"]
        d = f["model_weights/dense/dense/kernel:0"]
        assert d.shape == (6, 5)
        np.testing.assert_array_equal(np.asarray(d), k1)
        assert json.loads(f.attrs["model_config"]) == cfg and f.attrs["keras_version"] == "2.9.0"
        with pytest.raises(KeyError):
            f["model_weights/missing"]
    with Hdf5Archive(p) as ar:
        assert ar.getGroups() == ["model_weights"] and ar.getDataSets("model_weights", "dense", "dense") == ["bias:0", "kernel:0"]
        assert ar.readAttributeAsJson("model_config")["class_name"] == "Sequential"
        assert ar.readAttributeAsStringList("weight_names", "model_weights", "dense_1") == ["dense_1/kernel:0", "dense_1/bias:0"]
        np.testing.assert_array_equal(ar.readDataSet("bias:0", "model_weights", "dense_1", "dense_1"), b2)
        assert ar.hasAttribute("backend") and not ar.hasAttribute("nope")


def test_other_types_wide_groups_and_split_attributes(tmp_path):
    w = Hdf5Writer()
    for i in range(40):                                           # more children than one default leaf node holds
        w.dataset(f"g/d{i:02d}", np.arange(i + 1, dtype=np.int64))
    w.dataset("half", np.array([[1.5, -2.0]], dtype=np.float16))
    w.dataset("f64", np.linspace(0, 1, 7))
    w.dataset("u8", np.arange(5, dtype=np.uint8))
    w.dataset("empty", np.zeros((0, 3), dtype=np.float32))
    w.attr("g", "layer_names0", [b"a", b"bb"])
    w.attr("g", "layer_names1", [b"ccc"])
    w.attr("g", "ints", np.array([3, 1, 4], dtype=np.int32))
    w.attr("g", "scalar", np.float32(2.5))
    f = Hdf5File(w.tobytes())
    assert len(f["g"].keys()) == 40 and int(np.asarray(f["g/d07"]).sum()) == 28
    assert np.asarray(f["half"]).dtype == np.float16 and np.asarray(f["half"]).tolist() == [[1.5, -2.0]]
    np.testing.assert_allclose(np.asarray(f["f64"]), np.linspace(0, 1, 7))
    assert np.asarray(f["u8"]).dtype == np.uint8 and np.asarray(f["empty"]).shape == (0, 3)
    assert f["g"].attrs["ints"].tolist() == [3, 1, 4] and float(f["g"].attrs["scalar"]) == 2.5
    ar = Hdf5Archive(w.tobytes())
    assert ar.readAttributeAsStringList("layer_names", "g") == ["a", "bb", "ccc"]


def test_unsupported_structures_are_named():
    with pytest.raises(Hdf5FormatError, match="signature"):
        Hdf5File(b"not an hdf5 file at all" * 10)
    sb2 = b"\x89HDF\r\n\x1a\n" + bytes([2]) + b"\0" * 100
    with pytest.raises(Hdf5FormatError, match="superblock version 2"):
        Hdf5File(sb2)


def test_keras_full_model_file_imports(tmp_path):
    from deeplearning4j_b200.importers import KerasModelImport
    p, _, (k1, b1, k2, b2) = _keras_file(tmp_path)
    net = KerasModelImport.importKerasModelAndWeights(p)
    x = torch.tensor(np.random.default_rng(1).standard_normal((4, 6)).astype(np.float32))
    ref = torch.softmax(torch.tanh(x @ torch.tensor(k1) + torch.tensor(b1)) @ torch.tensor(k2) + torch.tensor(b2), -1)
    out = net.output(x)
    torch.testing.assert_close(out.t if hasattr(out, "t") else out, ref, rtol=1e-5, atol=1e-6)


def test_keras_json_plus_weights_only_file(tmp_path):
    from deeplearning4j_b200.importers import KerasModelImport
    p, cfg, (k1, b1, k2, b2) = _keras_file(tmp_path, full=False)
    net = KerasModelImport.importKerasSequentialModelAndWeights(json.dumps(cfg), p)
    x = torch.zeros(2, 6)
    out = net.output(x)
    ref = torch.softmax(torch.tanh(torch.tensor(b1)) @ torch.tensor(k2) + torch.tensor(b2), -1).expand(2, 3)
    torch.testing.assert_close(out.t if hasattr(out, "t") else out, ref, rtol=1e-5, atol=1e-6)


def test_chunked_and_compressed_datasets():
    g = np.random.default_rng(3)
    a = g.standard_normal((37, 21)).astype(np.float32)
    b = np.arange(1000, dtype=np.int32)
    w = Hdf5Writer()
    w.dataset("plain_chunks", a, chunks=(16, 8))                        # edge chunks are partly outside the dataset
    w.dataset("gzip", a, chunks=(10, 21), compression="gzip")
    w.dataset("shuffle_gzip", b, chunks=(256,), compression="gzip", shuffle=True)
    f = Hdf5File(w.tobytes())
    np.testing.assert_array_equal(np.asarray(f["plain_chunks"]), a)
    np.testing.assert_array_equal(np.asarray(f["gzip"]), a)
    np.testing.assert_array_equal(np.asarray(f["shuffle_gzip"]), b)
