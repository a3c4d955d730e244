"""``ModelSerializer``: DL4J zip checkpoints.

Entries, in the reference's order (``deeplearning4j-nn/.../util/ModelSerializer.java:60-65,
223-285``): ``configuration.json`` (Jackson JSON), ``coefficients.bin`` (``Nd4j.write`` of the
flat parameter row vector), ``noParams.marker`` when there are no parameters,
``updaterState.bin`` (flat updater state), ``normalizer.bin`` and ``objects/<key>`` extras.
Restore mirrors ``restoreMultiLayerNetwork`` ``:321-450`` / ``restoreComputationGraph``.
"""
from __future__ import annotations

import io
import json
import os
import pickle
import zipfile

import torch

from ..nd.ndarray import INDArray
from ..serde.binary import read_array, write_array

CONFIGURATION_JSON = "configuration.json"
COEFFICIENTS_BIN = "coefficients.bin"
UPDATER_BIN = "updaterState.bin"
NORMALIZER_BIN = "normalizer.bin"
PREPROCESSOR_BIN = "preprocessor.bin"
NO_PARAMS_MARKER = "noParams.marker"
OBJECTS_DIR = "objects/"
MAX_ENTRY_BYTES = 1 << 36     # zip-bomb guard (ModelSerializer.java:73-87)


def _flat_row(t: torch.Tensor) -> INDArray:
    return INDArray(t.detach().reshape(1, -1))


def _zinfo(name):
    zi = zipfile.ZipInfo(name, date_time=(1980, 1, 1, 0, 0, 0))   # deterministic archives
    zi.compress_type = zipfile.ZIP_DEFLATED
    return zi


class ModelSerializer:
    @staticmethod
    def writeModel(model, path_or_stream, saveUpdater=True, normalizer=None):
        own = isinstance(path_or_stream, (str, os.PathLike))
        f = open(path_or_stream, "wb") if own else path_or_stream
        try:
            with zipfile.ZipFile(f, "w", zipfile.ZIP_DEFLATED) as z:
                z.writestr(_zinfo(CONFIGURATION_JSON), model.conf.toJson().encode("utf-8"))
                if model.numParams() > 0:
                    bio = io.BytesIO()
                    write_array(_flat_row(model.flat_params), bio)
                    z.writestr(_zinfo(COEFFICIENTS_BIN), bio.getvalue())
                else:
                    z.writestr(_zinfo(NO_PARAMS_MARKER), b"")
                if saveUpdater and model.updater is not None and model.updater.state_size > 0:
                    bio = io.BytesIO()
                    write_array(_flat_row(model.updater.state), bio)
                    z.writestr(_zinfo(UPDATER_BIN), bio.getvalue())
                if normalizer is not None:
                    from ..data.normalizers import NormalizerSerializer
                    bio = io.BytesIO()
                    NormalizerSerializer.write(normalizer, bio)
                    z.writestr(_zinfo(NORMALIZER_BIN), bio.getvalue())
        finally:
            if own:
                f.close()

    @staticmethod
    def _open(path_or_stream):
        z = zipfile.ZipFile(path_or_stream, "r")
        for info in z.infolist():
            if info.file_size > MAX_ENTRY_BYTES:
                raise IOError(f"zip entry {info.filename} exceeds the {MAX_ENTRY_BYTES}-byte limit")
        return z

    @staticmethod
    def _restore(cls_factory, path_or_stream, loadUpdater, device=None):
        with ModelSerializer._open(path_or_stream) as z:
            names = set(z.namelist())
            if CONFIGURATION_JSON not in names:
                raise IOError("not a DL4J model zip: configuration.json missing")
            conf_json = z.read(CONFIGURATION_JSON).decode("utf-8")
            params = None
            if COEFFICIENTS_BIN in names:
                params = read_array(io.BytesIO(z.read(COEFFICIENTS_BIN))).t.reshape(-1)
            model = cls_factory(conf_json)
            if device is not None:
                model.device = torch.device(device)
            model.init(params, False)
            if loadUpdater and UPDATER_BIN in names:
                st = read_array(io.BytesIO(z.read(UPDATER_BIN))).t.reshape(-1)
                model._ensure_updater().setStateViewArray(st)
            return model

    @staticmethod
    def restoreMultiLayerNetwork(path_or_stream, loadUpdater=True, device=None):
        from .conf.neuralnet import MultiLayerConfiguration
        from .multilayer import MultiLayerNetwork
        return ModelSerializer._restore(lambda j: MultiLayerNetwork(MultiLayerConfiguration.fromJson(j)),
                                        path_or_stream, loadUpdater, device)

    @staticmethod
    def restoreComputationGraph(path_or_stream, loadUpdater=True, device=None):
        from .conf.graphconf import ComputationGraphConfiguration
        from .graph import ComputationGraph
        return ModelSerializer._restore(lambda j: ComputationGraph(ComputationGraphConfiguration.fromJson(j)),
                                        path_or_stream, loadUpdater, device)

    @staticmethod
    def restoreMultiLayerNetworkAndNormalizer(path, loadUpdater=True):
        return ModelSerializer.restoreMultiLayerNetwork(path, loadUpdater), ModelSerializer.restoreNormalizerFromFile(path)

    @staticmethod
    def restoreComputationGraphAndNormalizer(path, loadUpdater=True):
        return ModelSerializer.restoreComputationGraph(path, loadUpdater), ModelSerializer.restoreNormalizerFromFile(path)

    @staticmethod
    def addNormalizerToModel(path, normalizer):
        from ..data.normalizers import NormalizerSerializer
        bio = io.BytesIO()
        NormalizerSerializer.write(normalizer, bio)
        ModelSerializer._replace_entry(path, NORMALIZER_BIN, bio.getvalue())

    @staticmethod
    def restoreNormalizerFromFile(path):
        from ..data.normalizers import NormalizerSerializer
        with ModelSerializer._open(path) as z:
            if NORMALIZER_BIN not in z.namelist():
                return None
            return NormalizerSerializer.read(io.BytesIO(z.read(NORMALIZER_BIN)))

    @staticmethod
    def addObjectToFile(path, key, obj):
        ModelSerializer._replace_entry(path, OBJECTS_DIR + key, pickle.dumps(obj))

    @staticmethod
    def getObjectFromFile(path, key):
        with ModelSerializer._open(path) as z:
            return pickle.loads(z.read(OBJECTS_DIR + key))

    @staticmethod
    def listObjectsInFile(path):
        with ModelSerializer._open(path) as z:
            return [n[len(OBJECTS_DIR):] for n in z.namelist() if n.startswith(OBJECTS_DIR)]

    @staticmethod
    def _replace_entry(path, name, data):
        with zipfile.ZipFile(path, "r") as z:
            items = [(i.filename, z.read(i.filename)) for i in z.infolist() if i.filename != name]
        with zipfile.ZipFile(path, "w", zipfile.ZIP_DEFLATED) as z:
            for n, b in items:
                z.writestr(_zinfo(n), b)
            z.writestr(_zinfo(name), data)


class ModelGuesser:
    """``deeplearning4j-core/.../util/ModelGuesser.java``: load whatever the file holds."""

    @staticmethod
    def loadModelGuess(path):
        with zipfile.ZipFile(path, "r") as z:
            conf = json.loads(z.read(CONFIGURATION_JSON).decode("utf-8"))
        if "vertices" in conf:
            return ModelSerializer.restoreComputationGraph(path)
        return ModelSerializer.restoreMultiLayerNetwork(path)

    @staticmethod
    def loadConfigGuess(path):
        s = open(path).read()
        d = json.loads(s)
        if "vertices" in d:
            from .conf.graphconf import ComputationGraphConfiguration
            return ComputationGraphConfiguration.fromJson(s)
        from .conf.neuralnet import MultiLayerConfiguration
        return MultiLayerConfiguration.fromJson(s)
