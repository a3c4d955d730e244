"""Model hub access (``omnihub`` ``OmniHubUtils`` + per-framework namespaces): resolve a model by framework and name in the local
cache (``$OMNIHUB_HOME`` or ``~/.omnihub``), download it when it is missing, and load it into a SameDiff graph or a DL4J network.

This build has no network access, so the download step raises with the exact path where the file is expected; everything else
(cache layout ``<home>/<framework>/<file>``, loading by extension through the importers) works on files already present."""
from __future__ import annotations

import os


class OmniHubUtils:
    DEFAULT_HOME = os.path.join(os.path.expanduser("~"), ".omnihub")
    FRAMEWORKS = ("samediff", "dl4j", "onnx", "tensorflow", "keras", "pytorch", "huggingface")

    @staticmethod
    def getCacheDir():
        d = os.environ.get("OMNIHUB_HOME", OmniHubUtils.DEFAULT_HOME)
        os.makedirs(d, exist_ok=True)
        return d

    @staticmethod
    def modelPath(framework, fileName):
        if framework not in OmniHubUtils.FRAMEWORKS:
            raise ValueError(f"unknown framework '{framework}' (expected one of {OmniHubUtils.FRAMEWORKS})")
        return os.path.join(OmniHubUtils.getCacheDir(), framework, fileName)

    @staticmethod
    def downloadAndLoadFromZoo(framework, fileName, forceDownload=False):
        path = OmniHubUtils.modelPath(framework, fileName)
        if forceDownload or not os.path.exists(path):
            raise IOError(f"model '{fileName}' is not in the local cache and cannot be downloaded here (no network): place it at {path}")
        return path

    @staticmethod
    def loadSameDiffModel(fileName, forceDownload=False):
        from ..samediff import SameDiff
        path = OmniHubUtils.downloadAndLoadFromZoo("samediff", fileName, forceDownload)
        return SameDiff.load(path) if not path.endswith(".fb") else SameDiff.fromFlatFile(path)

    @staticmethod
    def loadNetwork(fileName, forceDownload=False):
        from ..nn import ModelGuesser
        return ModelGuesser.loadModelGuess(OmniHubUtils.downloadAndLoadFromZoo("dl4j", fileName, forceDownload))

    @staticmethod
    def loadForeign(framework, fileName, forceDownload=False):
        """ONNX / TensorFlow / Keras files through the importers."""
        from .. import importers
        path = OmniHubUtils.downloadAndLoadFromZoo(framework, fileName, forceDownload)
        if framework == "onnx":
            return importers.importOnnx(path)
        if framework == "tensorflow":
            return importers.importFrozenTF(path)
        if framework == "keras":
            return importers.KerasModelImport.importKerasModelAndWeights(path)
        raise ValueError(f"no importer for framework '{framework}'")
